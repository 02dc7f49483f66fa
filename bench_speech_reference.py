"""Reference arms of ``bench_speech.py``: the UNMODIFIED reference package under ``baseline/_ref`` on the speech configs.

Whisper-large-v2, fully sharded (config 5).  The reference has two Whisper paths.  Its own model class
(onmt/models/speech_recognizer/whisper.py) cannot run a forward pass: ``WhisperModel.forward`` stores an undefined name
(``output_dict['hidden'] = decoder_output`` at :100, the assignment above it is commented out), so every call raises
``NameError``.  The path that the reference's users run is the Hugging Face one (whisper/train_whisper.py): the model is
``MemoryEfficientWhisper`` (whisper/memory_efficient_whisper.py:237, a ``WhisperForConditionalGeneration`` with the
reference's fused LayerNorm / cross-entropy where its extensions load, PyTorch otherwise), trained under FSDP
``full_shard auto_wrap`` with the encoder and decoder layer classes as the wrapped units (train_whisper.py:597-600),
AdamW, gradient-norm clipping at 1.0 (:584).  This arm builds that model class with
random weights of the large-v2 sizes (no checkpoint is reachable), wraps it the same way with torch FSDP - which is what
the Hugging Face trainer does with those arguments - and runs the same step: forward with labels, backward,
``clip_grad_norm_``, ``AdamW.step``.  The trainer object itself is not used because it needs a ``datasets`` corpus.

wav2vec2-large + mBART-50 (config 4) has no reference arm here: the reference's wrapper module imports ``omegaconf``
at load time and passes the checkpoint's configuration through ``OmegaConf.create`` / ``set_struct``
(onmt/models/speech_recognizer/wav2vec2.py:11, 79-81); that package is not installed and not in the offline
wheelhouse, and standing in for it would put code of this repository on the reference's path.

None of this framework's models, kernels or engine is imported here.
"""
from __future__ import annotations

import functools
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference_whisper():
    import bench_reference as br
    ok, why = br.reference_available()
    if not ok:
        raise RuntimeError(why)
    br.import_reference()
    script_dir = os.path.join(br.REF, "whisper")        # the reference's scripts import their siblings as top-level modules
    if script_dir not in sys.path:
        sys.path.insert(0, script_dir)
    import memory_efficient_whisper as mw
    return mw


class WhisperReferenceRunner:
    """``MemoryEfficientWhisper`` under FSDP full-shard auto-wrap, one AdamW step per call."""

    def __init__(self, sizes: dict, device, rank: int, world: int, attn: str = "sdpa"):
        from transformers import WhisperConfig
        mw = _import_reference_whisper()
        self.device = torch.device(device)
        cuda = self.device.type == "cuda"
        cfg = WhisperConfig(vocab_size=sizes["vocab"], num_mel_bins=sizes["n_mels"], d_model=sizes["dim"],
                            encoder_layers=sizes["layers"], decoder_layers=sizes["layers"],
                            encoder_attention_heads=sizes["heads"], decoder_attention_heads=sizes["heads"],
                            encoder_ffn_dim=sizes["ffn"], decoder_ffn_dim=sizes["ffn"],
                            max_source_positions=sizes["frames"] // 2, max_target_positions=448, dropout=0.1, attention_dropout=0.1,
                            pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)
        cfg._attn_implementation = attn
        model = mw.MemoryEfficientWhisper(cfg)
        # create_whisper_model (:439-452) would now swap every encoder layer for MemoryEfficientWhisperEncoderLayer.  That
        # class's forward(hidden_states, attention_mask, layer_head_mask, output_attentions) was written for an older
        # transformers release; the installed 5.5 calls encoder layers with other keywords and the swapped layer raises
        # "unexpected keyword argument 'head_mask'".  The stock encoder layers of the model class are kept instead (the
        # swap only changes how the residual sums are stored), and they are the FSDP wrapping unit below.
        enc_layer_cls = type(model.model.encoder.layers[0])
        self.n_params = sum(p.numel() for p in model.parameters())
        dtype = torch.bfloat16 if cuda else torch.float32
        model = model.to(dtype)
        model.train()
        self.dtype = dtype
        self.world = world
        self.path = "MemoryEfficientWhisper (attention: %s)" % attn
        if cuda and (world > 1 or os.environ.get("NMTG_REF_FSDP_SINGLE", "1") == "1"):
            from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
            from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy
            from transformers.models.whisper.modeling_whisper import WhisperDecoderLayer
            import torch.distributed as dist
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29531")
                dist.init_process_group("nccl", rank=0, world_size=1, device_id=self.device)
                self._own_group = True
            policy = functools.partial(transformer_auto_wrap_policy,
                                       transformer_layer_cls={enc_layer_cls, WhisperDecoderLayer})
            model = FSDP(model, auto_wrap_policy=policy, device_id=self.device.index, use_orig_params=True)
            self.path += " + torch FSDP full_shard auto_wrap"
            self.fsdp = True
        else:
            model = model.to(self.device)
            self.fsdp = False
        self.model = model
        self.optim = torch.optim.AdamW(model.parameters(), lr=1e-5, weight_decay=0.01)

    def collate(self, feats, targets):
        """feats: list of [frames, n_mels] tensors (all 30 s windows); targets: list of id tensors (BOS ... EOS)."""
        x = torch.stack([f.t() for f in feats]).to(self.dtype)                 # [B, n_mels, frames]
        T = max(int(t.numel()) for t in targets)
        labels = torch.full((len(targets), T - 1), -100, dtype=torch.long)
        for i, t in enumerate(targets):
            labels[i, :t.numel() - 1] = t[1:]
        pin = self.device.type == "cuda"
        return (x.pin_memory() if pin else x), (labels.pin_memory() if pin else labels), int(sum(t.numel() - 1 for t in targets))

    @staticmethod
    def h2d_bytes(batch):
        return batch[0].numel() * batch[0].element_size() + batch[1].numel() * 8

    def step(self, batch):
        x, labels, _ = batch
        x = x.to(self.device, non_blocking=True)
        labels = labels.to(self.device, non_blocking=True)
        out = self.model(input_features=x, labels=labels)
        loss = out.loss
        loss.backward()
        if self.fsdp:
            self.model.clip_grad_norm_(1.0)
        else:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.optim.step()
        self.optim.zero_grad(set_to_none=True)
        return loss.detach()

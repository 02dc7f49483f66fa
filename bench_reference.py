"""Reference arm of the benchmark: the UNMODIFIED reference package (installed under ``baseline/_ref``)
driven through its own public pieces in the order its trainer uses them
(onmt/train_utils/mp_trainer.py:202-387 set-up, :743-1019 step):

    build_model -> NMTLossFunc -> optimize_model -> init_model_parameters -> .cuda() -> onmt.Optim ->
    DistributedDataParallel (world size > 1) -> per step: Batch.cuda, autocast(bf16) forward, loss,
    GradScaler.scale(loss).backward(), all_reduce(word count), unscale_, clip_grad_norm, optim.step,
    scaler.update, zero_grad.

None of this framework's models, kernels or engine is imported here.  The only additions are two stub
modules for optional audio dependencies that are not installed (``soundfile``, ``kaldiio``), injected
through ``sys.modules`` without touching the reference's files.  The reference's own trainer class cannot
be used directly because it needs on-disk datasets; its step is restated with the same calls.
"""
from __future__ import annotations

import argparse
import importlib.machinery
import os
import sys
import types
import warnings

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "baseline", "_ref")


def reference_available():
    if not os.path.isdir(os.path.join(REF, "onmt")):
        return False, "reference is not installed under baseline/_ref"
    if not os.path.exists(os.path.join(REF, "options.py")):
        return False, "baseline/_ref/options.py is missing (the reference's setup.py does not install it)"
    return True, ""


def import_reference():
    warnings.filterwarnings("ignore")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    for name in ("soundfile", "kaldiio", "kaldiio.python_wave"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__spec__ = importlib.machinery.ModuleSpec(name, None)
            sys.modules[name] = m
    sys.modules["kaldiio"].__path__ = []
    sys.modules["soundfile"].read = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("soundfile is a stub"))
    import onmt  # noqa: F401
    import options
    return onmt, options


def make_opt(options, argv):
    p = argparse.ArgumentParser()
    options.make_parser(p)
    opt = p.parse_args(argv)
    return options.backward_compatible(opt)


def transformer_big_argv(tiny=False):
    if tiny:
        size = ["-layers", "2", "-model_size", "256", "-n_heads", "4", "-inner_size", "1024"]
    else:
        size = ["-layers", "6", "-model_size", "1024", "-n_heads", "16", "-inner_size", "4096"]
    return ["-data", "none", "-model", "transformer"] + size + [
        "-dropout", "0.1", "-attn_dropout", "0.1", "-emb_dropout", "0.1", "-ffn_activation", "relu", "-tie_weights",
        "-join_embedding", "-label_smoothing", "0.1", "-optim", "adam", "-weight_decay", "0.01", "-learning_rate", "2.0",
        "-update_method", "noam", "-warmup_steps", "4000", "-max_grad_norm", "5", "-fp16", "-bf16",
        "-batch_size_words", "8192"]


class ReferenceRunner:
    """Builds the reference model / loss / optimiser once and exposes ``step(host_batch)``."""

    def __init__(self, vocab_size, device, rank=0, world_size=1, tiny=False, argv_extra=()):
        onmt, options = import_reference()
        self.onmt = onmt
        from onmt.model_factory import build_model, init_model_parameters, optimize_model
        from onmt.modules.loss import NMTLossFunc
        from onmt.constants import add_tokenidx
        self.opt = opt = make_opt(options, transformer_big_argv(tiny) + list(argv_extra))     # later flags win
        d = onmt.Dict(["<blank>", "<unk>", "<s>", "</s>"])
        for i in range(vocab_size - 4):
            d.add("w%d" % i)
        dicts = {"src": d, "tgt": d, "langs": {"src": 0, "tgt": 1}, "atbs": {"nothingness": 0}}
        onmt.constants = add_tokenidx(opt, onmt.constants, dicts)
        dicts["tgt_pad"] = onmt.constants.TGT_PAD
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.world_size = world_size
        model = build_model(opt, dicts, False, onmt.constants)
        self.loss_function = NMTLossFunc(opt.model_size, d.size(), label_smoothing=opt.label_smoothing,
                                         mirror=opt.mirror_loss, padding_idx=dicts["tgt_pad"])
        optimize_model(model, distributed=world_size > 1)
        init_model_parameters(model, opt)
        if self.cuda:
            self.loss_function = self.loss_function.cuda(device=self.device)
            model = model.cuda(device=self.device)
        self.grad_scaler = torch.cuda.amp.GradScaler() if self.cuda else None
        self.optim = onmt.Optim(opt)
        self.optim.set_parameters(model.parameters())
        self.raw_model = model
        if world_size > 1:
            model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[self.device.index],
                                                              output_device=self.device.index,
                                                              find_unused_parameters=opt.find_unused_parameters)
        self.model = model
        self.num_words = torch.zeros(1, device=self.device)
        self.n_params = sum(p.numel() for p in self.raw_model.parameters() if p.requires_grad)

    def collate(self, src_list, tgt_list):
        """The reference's own collate_fn + Batch on host tensors (pinned when CUDA is present)."""
        from onmt.data.dataset import collate_fn
        light = collate_fn(src_list, tgt_list, None, None, None, None, False, False, src_type="text",
                           src_pad=self.onmt.constants.SRC_PAD, tgt_pad=self.onmt.constants.TGT_PAD)
        return light.pin_memory() if self.cuda else light

    @staticmethod
    def h2d_bytes(batch):
        return sum(v.numel() * v.element_size() for v in batch.tensors.values() if isinstance(v, torch.Tensor))

    def step(self, batch):
        """One update, mirroring Trainer.train_epoch for update_frequency 1.  Returns the loss tensor."""
        from onmt.utils import clip_grad_norm
        import torch.distributed as dist
        from onmt.data.dataset import rewrap
        opt = self.opt
        batch = rewrap(batch)          # LightBatch -> Batch, as prepare_sample does
        if self.cuda:
            batch.cuda(fp16=False, device=self.device)
        targets = batch.get("target_output")
        bf16 = self.cuda
        with torch.autocast(device_type=self.device.type, enabled=bool(opt.fp16) and self.cuda, dtype=torch.bfloat16):
            tgt_mask = batch.get("target_input_selfattn_mask")
            outputs = self.model(batch, streaming=False, target_mask=tgt_mask, zero_encoder=opt.zero_encoder,
                                 mirror=opt.mirror_loss, streaming_state=None, nce=opt.nce, pretrained_layer_states=None,
                                 adv_ptb_grad=False, checkpointing_ffn=opt.checkpointing_ffn,
                                 checkpointing_cross_attn=opt.checkpointing_cross_attn,
                                 checkpointing_self_attn=opt.checkpointing_self_attn, ctc_loss_function=None,
                                 ctc_labels=targets, grad_scaler=self.grad_scaler, ctc_coeff=0.0)
            outputs["tgt_mask"] = tgt_mask
            loss_dict = self.loss_function(outputs, targets, model=self.raw_model)
            full_loss = loss_dict["loss"]
        if self.grad_scaler is not None:
            self.grad_scaler.scale(full_loss).backward()
        else:
            full_loss.backward()
        self.raw_model.post_backward(output_dict=outputs)
        self.num_words.add_(batch.tgt_size)
        if self.world_size > 1:
            dist.all_reduce(self.num_words, op=dist.ReduceOp.SUM)
        if self.grad_scaler is not None:
            self.grad_scaler.unscale_(self.optim.optimizer)
        clip_grad_norm(self.raw_model.parameters(), opt.max_grad_norm)
        if self.grad_scaler is not None:
            self.optim.step(scaler=self.grad_scaler)
            self.grad_scaler.update()
        else:
            self.optim.step(scaler=None)
        self.optim.zero_grad(set_to_none=opt.true_zero_grad)
        self.num_words.zero_()
        return loss_dict["data"] if isinstance(loss_dict["data"], torch.Tensor) else full_loss.detach()


if __name__ == "__main__":
    # CPU self-check of the harness on a tiny model (no timing)
    ok, why = reference_available()
    if not ok:
        print(why)
        sys.exit(0)
    import numpy as np
    r = ReferenceRunner(2000, "cpu", tiny=True)
    rng = np.random.RandomState(0)
    src = [torch.from_numpy(rng.randint(4, 2000, size=12).astype(np.int64)) for _ in range(8)]
    tgt = [torch.from_numpy(np.concatenate([[2], rng.randint(4, 2000, size=15), [3]]).astype(np.int64)) for _ in range(8)]
    for i in range(3):
        b = r.collate(src, tgt)
        print("reference loss/token", float(r.step(b)) / b.tensors["tgt_size"])

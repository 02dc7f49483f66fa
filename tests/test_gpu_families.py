"""Every model family trains one step and decodes on the GPU through the fused ops (bf16 working copies)."""
import copy
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

from nmtgminor_b200 import ops
from nmtgminor_b200.data.synthetic import synthetic_audio_batch, synthetic_dict, token_budget_batches
from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
from nmtgminor_b200.models.factory import build_classifier, build_language_model, build_model
from nmtgminor_b200.options import default_options
from nmtgminor_b200.parallel.flat import FlatParameterStore

COMMON = ["-model_size", "128", "-layers", "2", "-n_heads", "2", "-inner_size", "256", "-dropout", "0.1", "-attn_dropout", "0.1",
          "-ffn_activation", "relu", "-label_smoothing", "0.1"]


@pytest.fixture(scope="module")
def dicts():
    d = synthetic_dict(120)
    return {"src": d, "tgt": d, "langs": {"en": 0, "de": 1}}


def _to_gpu(model):
    store = FlatParameterStore(model, "cuda")
    for b in model.buffers():
        b.data = b.data.cuda()
    return store


def _step_and_decode(model, batch, decode=True):
    store = _to_gpu(model)
    gb = copy.deepcopy(batch).cuda("cuda")
    model.train()
    out = model(gb)
    assert torch.isfinite(out["loss"]).all()
    out["loss"].backward()
    store.gather_autograd_grads()
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    assert torch.isfinite(store.grad).all() and float(store.grad.abs().sum()) > 0
    if decode:
        model.eval()
        hyps = beam_search(model, gb, BeamConfig(beam_size=2, max_len=5))
        assert len(hyps) == batch.size and all(h[0].tokens for h in hyps)
        assert ops.check_status() == 0


@pytest.mark.parametrize("name,extra", [
    ("transformer", ["-death_rate", "0.1", "-variational_dropout"]), ("relative_transformer", []), ("universal_transformer", []),
    ("multilingual_translator", ["-multilingual_adapter", "-adapter_bottleneck_size", "16"]), ("LSTM", []),
    ("discourse_translator", []), ("pretrain_transformer", ["-enc_pretrained_model", "mbart50", "-dec_pretrained_model", "mbart50"]),
    ("pretrain_transformer", ["-enc_pretrained_model", "deltalm", "-dec_pretrained_model", "deltalm"]),
    ("dlcl_transformer", []), ("parallel_transformer", []), ("fctransformer", []), ("unified_transformer", []),
    ("transformer", ["-depthwise_conv", "-conv_kernel", "5", "-no_ffn", "-macaron"]), ("transformer", ["-favor_attention"]),
    ("relative_transformer", ["-absolute_position_encoding"]),
])
def test_text_families_on_gpu(dicts, name, extra):
    torch.manual_seed(0)
    model = build_model(default_options(["-model", name] + COMMON + extra), dicts)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    _step_and_decode(model, batch)


def test_speech_families_on_gpu(dicts, tmp_path):
    torch.manual_seed(1)
    def cfg(name, **kw):
        p = tmp_path / name
        p.write_text(json.dumps(kw))
        return str(p)
    enc = cfg("enc.json", encoder_embed_dim=128, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=256)
    dec = cfg("dec.json", d_model=128, decoder_layers=2, decoder_attention_heads=2, decoder_ffn_dim=256, vocab_size=120, pad_token_id=0)
    wsp = cfg("whisper.json", d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=256,
              num_mel_bins=80, max_source_positions=128, max_target_positions=64, vocab_size=120, pad_token_id=0)
    cases = [
        (["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50", "-ctc_loss", "0.3"],
         synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "wav2vec2_transformer", "-enc_config_file", enc], synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-enc_pretrained_model", "wavlm"],
         synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "whisper", "-dec_config_file", wsp], synthetic_audio_batch(2, 120, "feats", n_feats=80, fixed_frames=120)),
        (["-model", "speech_transformer", "-input_size", "40", "-cnn_downsampling"], synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)),
        (["-model", "conformer", "-input_size", "40"], synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)),
        (["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-branchformer", "-conv_kernel", "7"],
         synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-no_decoder"], synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "speech_transformer", "-input_size", "40", "-multilingual_linear_projection", "-depthwise_conv"],
         synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)),
    ]
    for argv, batch in cases:
        model = build_model(default_options(argv + COMMON), dicts)
        if "-multilingual_linear_projection" in argv:
            batch.tensors["source_lang"] = torch.tensor([0])
        _step_and_decode(model, batch, decode="-no_decoder" not in argv)
        if "-no_decoder" in argv:
            hyps = model.eval().ctc_greedy(copy.deepcopy(batch).cuda("cuda"))
            assert len(hyps) == batch.size and ops.check_status() == 0


def test_language_model_and_classifier_on_gpu(dicts):
    torch.manual_seed(2)
    lm = build_language_model(default_options(["-model", "transformer_xl_lm"] + COMMON), dicts)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    _step_and_decode(lm, batch, decode=False)

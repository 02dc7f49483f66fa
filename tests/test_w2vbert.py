"""w2v-BERT / Conformer-Shaw family on CPU: shapes, the Shaw position term against a direct restatement, causality of the
convolution, the quantiser and the two pre-training losses."""
import json
from types import SimpleNamespace

import torch

from nmtgminor_b200.models.layers import pack_padded
from nmtgminor_b200.models.w2vbert import (ConformerShawEncoder, GumbelVectorQuantizer, ShawConvolution,
                                           ShawRelPosSelfAttention, W2VBertModel, build_w2vbert_encoder, w2vbert_arch)


def _audio(B=3, T=64, F=80, lengths=(64, 50, 40)):
    src = torch.zeros(T, B, 1 + F)
    for b, L in enumerate(lengths):
        src[:L, b, 0] = 1
        src[:L, b, 1:] = torch.randn(L, F)
    return src


def test_presets():
    big, small = w2vbert_arch("600m"), w2vbert_arch("300m")
    assert (big.encoder.layers, big.encoder.model_dim, big.encoder.feature_dim, big.num_bert_layers) == (24, 1024, 160, 16)
    assert small.encoder.layers == 12 and big.num_codebook_entries == 1024 and big.temporal_mask_span == 10


def test_shaw_attention_matches_direct_formula():
    torch.manual_seed(0)
    att = ShawRelPosSelfAttention(32, 4, max_left=3, max_right=1).eval()
    x = torch.randn(2, 9, 32)
    lengths = torch.tensor([9, 6])
    packed, seqs = pack_padded(x, lengths)
    got = att(packed, seqs)
    outs = []
    for b, L in enumerate(lengths.tolist()):
        qkv = att.qkv(x[b, :L])
        q, k, v = (t.view(L, 4, 8).transpose(0, 1) for t in qkv.split(32, -1))
        scores = torch.zeros(4, L, L)
        for i in range(L):
            for j in range(L):
                r = att.rel_k.weight[min(max(j - i, -3), 1) + 3]
                scores[:, i, j] = (q[:, i] * (k[:, j] + r)).sum(-1) / 8 ** 0.5
        outs.append(att.out((scores.softmax(-1) @ v).transpose(0, 1).reshape(L, 32)))
    assert torch.allclose(got, torch.cat(outs), atol=1e-4)


def test_causal_convolution_sees_no_future():
    torch.manual_seed(0)
    conv = ShawConvolution(16, 5, causal=True).eval()
    x = torch.randn(1, 20, 16)
    valid = torch.ones(1, 20)
    y0 = conv(x, valid)
    x2 = x.clone()
    x2[0, 12:] += 1.0
    y1 = conv(x2, valid)
    assert torch.allclose(y0[0, :12], y1[0, :12], atol=1e-6) and not torch.allclose(y0[0, 12:], y1[0, 12:])


def test_encoder_shapes_and_padding_invariance():
    torch.manual_seed(0)
    enc = ConformerShawEncoder(w2vbert_arch("test").encoder).eval()
    src = _audio()
    out, seqs = enc(src)
    assert out.shape == (32 + 25 + 20, 64) and seqs.cu.tolist() == [0, 32, 57, 77]
    alone, _ = enc(src[:50, 1:2])
    assert torch.allclose(out[32:57], alone, atol=1e-4)


def test_quantizer_train_and_eval():
    torch.manual_seed(0)
    vq = GumbelVectorQuantizer(20, 12, groups=3, entries=8)
    x = torch.randn(50, 20)
    q, ids, div, ppl = vq(x)
    assert q.shape == (50, 12) and ids.shape == (50, 3) and 0 <= float(div) <= 1 and vq.updates == 1
    vq.eval()
    q2, ids2, _, _ = vq(x)
    want = torch.cat([vq.codebook[g, ids2[:, g]] for g in range(3)], -1)
    assert torch.equal(q2, want)
    assert vq.temperature < 2.0


def test_pretraining_losses_backward():
    torch.manual_seed(0)
    model = W2VBertModel(w2vbert_arch("test"))
    gen = torch.Generator().manual_seed(1)
    out = model(_audio(), generator=gen)
    assert out["num_masked"] > 0 and torch.isfinite(out["loss"])
    out["loss"].backward()
    for name in ("masker.mask_vector", "quantizer.codebook", "final_proj.weight", "bert_proj.weight",
                 "encoder.layers.0.attn.rel_k.weight", "encoder.layers.2.ffn2.fc2.weight"):
        g = dict(model.named_parameters())[name].grad
        assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0, name


def test_builder_reads_config_file(tmp_path):
    path = tmp_path / "enc.json"
    path.write_text(json.dumps({"model_dim": 48, "num_encoder_layers": 2, "num_encoder_attn_heads": 4, "ffn_inner_dim": 96}))
    opt = SimpleNamespace(enc_pretrained_model="w2vbert", dropout=0.1, attn_dropout=0.0, death_rate=0.0, model_size=32,
                          layers=1, n_heads=2, inner_size=64, input_size=40)
    enc = build_w2vbert_encoder(opt, json.loads(path.read_text()))
    assert len(enc.layers) == 2 and enc.dim == 48 and enc.cfg.dropout == 0.1 and enc.cfg.feature_dim == 80
    plain = build_w2vbert_encoder(opt)                     # no file: the sizes of the command line
    assert len(plain.layers) == 1 and plain.dim == 32 and plain.cfg.heads == 2
    assert w2vbert_arch("300m").encoder.layers == 12       # a name with 300m / 600m selects the preset instead

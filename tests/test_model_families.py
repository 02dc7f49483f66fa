"""Every model family of the factory builds, trains one step and (where it decodes) runs beam search on CPU."""
import json
import math

import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_audio_batch, synthetic_dict, token_budget_batches
from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
from nmtgminor_b200.models import factory
from nmtgminor_b200.models.factory import build_classifier, build_language_model, build_model
from nmtgminor_b200.options import default_options

COMMON = ["-model_size", "64", "-layers", "2", "-n_heads", "2", "-inner_size", "128", "-dropout", "0.1", "-attn_dropout", "0.0",
          "-ffn_activation", "relu", "-label_smoothing", "0.1"]
REFERENCE_MODEL_NAMES = ["transformer", "stochastic_transformer", "relative_transformer", "universal_transformer",
                         "multilingual_translator", "translator", "speech_transformer", "conformer", "hybrid_transformer", "LSTM", "lstm",
                         "discourse_speech_transformer", "discourse_translator", "wav2vec2_transformer", "wav2vec2_bert",
                         "quantize_wav2vec2_bert", "quantize_wav2vec2_mbart50", "pretrain_transformer", "whisper"]


@pytest.fixture(scope="module")
def dicts():
    d = synthetic_dict(120)
    return {"src": d, "tgt": d, "langs": {"en": 0, "de": 1}}


def _cfg(tmp_path, name, **kw):
    p = tmp_path / name
    p.write_text(json.dumps(kw))
    return str(p)


def test_registry_covers_the_reference_model_names():
    factory._load_builders()
    missing = [n for n in REFERENCE_MODEL_NAMES if n not in factory._REGISTRY]
    assert not missing, missing


@pytest.mark.parametrize("name,extra", [
    ("transformer", ["-death_rate", "0.1"]), ("relative_transformer", []), ("universal_transformer", []),
    ("multilingual_translator", ["-multilingual_adapter", "-adapter_bottleneck_size", "16"]), ("LSTM", []),
    ("discourse_translator", []), ("pretrain_transformer", ["-enc_pretrained_model", "mbart50", "-dec_pretrained_model", "mbart50"]),
    ("pretrain_transformer", ["-enc_pretrained_model", "deltalm", "-dec_pretrained_model", "deltalm"]),
])
def test_text_families_train_and_decode(dicts, name, extra):
    torch.manual_seed(0)
    model = build_model(default_options(["-model", name] + COMMON + extra), dicts)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    out = model(batch)
    assert torch.isfinite(out["loss"]).all()
    out["loss"].backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.parameters())
    model.eval()
    hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=5))
    assert len(hyps) == batch.size and all(h[0].tokens for h in hyps)


def test_speech_families(dicts, tmp_path):
    torch.manual_seed(1)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=2, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    wsp = _cfg(tmp_path, "whisper.json", d_model=64, encoder_layers=2, decoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=128,
               num_mel_bins=80, max_source_positions=128, max_target_positions=64, vocab_size=120, pad_token_id=0)
    cases = [
        (["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50", "-ctc_loss", "0.3"],
         synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "wav2vec2_transformer", "-enc_config_file", enc], synthetic_audio_batch(2, 120, "wav", 3000, 6000)),
        (["-model", "whisper", "-dec_config_file", wsp], synthetic_audio_batch(2, 120, "feats", n_feats=80, fixed_frames=120)),
        (["-model", "speech_transformer", "-input_size", "40", "-cnn_downsampling"], synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)),
        (["-model", "conformer", "-input_size", "40"], synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)),
    ]
    for argv, batch in cases:
        model = build_model(default_options(argv + COMMON), dicts)
        out = model(batch)
        assert torch.isfinite(out["loss"]).all(), argv
        out["loss"].backward()
        model.eval()
        hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=4))
        assert len(hyps) == 2
    # wav2vec2: frame count follows the 320x conv stride, extractor frozen by default
    w2v = build_model(default_options(cases[0][0] + COMMON), dicts)
    ctx, seqs = w2v.encode(cases[0][1])
    lens = (cases[0][1].get("source")[:, :, 0] > 0).sum(0)
    assert (seqs.cu[1:] - seqs.cu[:-1]).tolist() == w2v.encoder.extractor.output_lengths(lens).tolist()
    assert all(not p.requires_grad for p in w2v.encoder.extractor.parameters())


def test_language_model_and_classifier(dicts):
    lm = build_language_model(default_options(["-model", "transformer_xl", "-max_memory_size", "8"] + COMMON), dicts)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    stream = lm.init_stream()
    l1 = lm(batch, streaming_state=stream)["loss"]
    l1.backward()
    assert stream.mems[0] is not None and stream.mems[0].shape[1] <= 8
    clf = build_classifier(default_options(COMMON), dicts)
    batch.tensors["labels"] = torch.randint(0, 5, (batch.size,))
    out = clf(batch)
    out["loss"].backward()
    assert out["logits"].shape == (batch.size, 120)


def test_state_space_encoder_and_backend_selection(dicts):
    from nmtgminor_b200.models.mssm import TiedStateSpaceModel
    torch.manual_seed(0)
    ssm = TiedStateSpaceModel(8, heads=2, state=4, channels=1)
    k = ssm.kernel(16)
    assert k.shape == (1, 16, 8) and torch.isfinite(k).all()
    # causal convolution: an impulse at t = 3 produces the kernel shifted by 3 (plus the skip term)
    u = torch.zeros(1, 16, 8)
    u[0, 3] = 1.0
    y = ssm(u)
    assert torch.allclose(y[0, :3], torch.zeros(3, 8), atol=1e-4)
    assert torch.allclose(y[0, 4:10], k[0, 1:7], atol=1e-4)
    for name, kind, feats in (("s4", "feats", 40), ("w2v-bert", "feats", 40), ("hubert_base", "wav", 1)):
        argv = ["-model", "wav2vec2_transformer", "-enc_pretrained_model", name, "-input_size", str(feats)] + COMMON
        model = build_model(default_options(argv), dicts)
        batch = (synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=feats) if kind == "feats"
                 else synthetic_audio_batch(2, 120, "wav", 3000, 5000))
        out = model(batch)
        assert torch.isfinite(out["loss"]).all(), name
        out["loss"].backward()


def test_ctc_compression_merges_runs(dicts, tmp_path):
    from nmtgminor_b200.models.layers import PackedSeqs
    from nmtgminor_b200.models.pretrained import ctc_compress
    ctx = torch.arange(7, dtype=torch.float32)[:, None].repeat(1, 2)
    cu = torch.tensor([0, 4, 7], dtype=torch.int32)
    seqs = PackedSeqs(torch.zeros(7, dtype=torch.long), torch.arange(7), cu, 4)
    logits = torch.full((7, 3), -5.0)
    for i, sym in enumerate([1, 1, 2, 2, 2, 0, 0]):      # runs: [0,1] [2,3] | [4] [5,6]  (the boundary splits the run of 2s)
        logits[i, sym] = 5.0
    out, new = ctc_compress(ctx, seqs, logits, "avg")
    assert new.cu.tolist() == [0, 2, 4]
    assert torch.allclose(out[:, 0], torch.tensor([0.5, 2.5, 4.0, 5.5]))
    enc = _cfg(tmp_path, "enc2.json", encoder_embed_dim=64, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    model = build_model(default_options(["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-ctc_loss", "0.3", "-ctc_compress", "avg"] + COMMON), dicts)
    out = model(synthetic_audio_batch(2, 120, "wav", 3000, 5000))
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and out["src"].cu[-1] <= out["context_packed"].shape[0]


def test_wavlm_gated_relative_position_bias(dicts, tmp_path):
    """``-enc_pretrained_model wavlm`` puts the gated relative-position attention in every encoder layer; the table is
    owned by the first layer, the sub-layer matches a direct statement of the formula, and it trains."""
    from nmtgminor_b200.models.speech_encoders import GatedRelPosSelfAttention
    from nmtgminor_b200.models.layers import PackedSeqs
    torch.manual_seed(5)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128,
               num_buckets=32, max_distance=64)
    model = build_model(default_options(["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-enc_pretrained_model", "wavlm"]
                                        + COMMON), dicts)
    attns = [l.attn for l in model.encoder.layers]
    assert all(isinstance(a, GatedRelPosSelfAttention) for a in attns)
    assert attns[0].relative_attention_bias is not None and attns[1].relative_attention_bias is None
    out = model(synthetic_audio_batch(2, 120, "wav", 3000, 6000))
    assert torch.isfinite(out["loss"]).all()
    out["loss"].backward()
    assert attns[0].relative_attention_bias.weight.grad.abs().sum() > 0 and attns[1].grep_linear.weight.grad.abs().sum() > 0

    # direct statement for one sequence
    a = attns[0].eval()
    T, H, h = 9, 64, 2
    x = torch.randn(T, H)
    seqs = PackedSeqs.from_padded(torch.ones(1, T, dtype=torch.long), torch.tensor([T]))
    got = a(x, seqs)
    qkv = a.qkv(x)
    q, k, v = (t.view(T, h, H // h).transpose(0, 1) for t in qkv.split(H, -1))
    pos = torch.arange(T)
    bias = a.relative_attention_bias(a._buckets(pos[None, :] - pos[:, None])).permute(2, 0, 1)
    g = torch.sigmoid(a.grep_linear(q).view(h, T, 2, 4).sum(-1))
    gate = g[..., :1] * (g[..., 1:] * a.grep_a[0] - 1.0) + 2.0
    p = torch.softmax(q @ k.transpose(1, 2) / (H // h) ** 0.5 + gate * bias, -1)
    want = a.out((p @ v).transpose(0, 1).reshape(T, H))
    assert torch.allclose(got, want, atol=1e-5)
    # buckets: symmetric halves, exact for small offsets, saturating for large ones
    b = a._buckets(torch.tensor([0, 1, -1, 5, -5, 1000, -1000]))
    assert b[0] == 0 and b[1] == 16 + 1 and b[2] == 1 and b[5] == 31 and b[6] == 15


def test_model_contract_extras(dicts):
    """Output keys trainers of the reference read (``src_mask``, ``target_mask``, ``softmaxed``) and encoder transplant."""
    torch.manual_seed(7)
    opt = default_options(["-model", "transformer"] + COMMON)
    a, b = build_model(opt, dicts), build_model(opt, dicts)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    out = a(batch, return_logits=True)
    T = batch.get("source").shape[0]
    assert out["src_mask"].shape == (batch.size, T) and out["src_mask"].dtype == torch.bool
    assert torch.equal(out["src_mask"], batch.get("src_selfattn_mask")) and out["softmaxed"] is False
    assert out["logprobs"].shape[:2] == batch.get("target_input").shape
    assert not torch.equal(a.encoder.layers[0].ffn.fc1.weight, b.encoder.layers[0].ffn.fc1.weight)
    b.load_encoder_weights(a)
    assert torch.equal(a.encoder.layers[0].ffn.fc1.weight, b.encoder.layers[0].ffn.fc1.weight)
    b.load_encoder_weights({k: torch.zeros_like(v) for k, v in a.state_dict().items()})
    assert float(b.encoder.layers[0].ffn.fc1.weight.abs().sum()) == 0 and float(b.decoder.layers[0].ffn.fc1.weight.abs().sum()) > 0
    assert a.init_stream() is None


def test_ctc_head_on_the_auxiliary_target(dicts):
    from nmtgminor_b200.data.synthetic import synthetic_dict
    torch.manual_seed(0)
    aux = synthetic_dict(23)
    argv = ["-model", "speech_transformer", "-input_size", "40", "-ctc_loss", "0.5"] + COMMON
    model = build_model(default_options(argv), {**dicts, "aux_tgt": aux})
    assert model.ctc_linear.out_features == aux.size() and model.ctc_on_aux
    batch = synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40)
    B = batch.get("target_output").shape[1]
    full = torch.zeros(B, 6, dtype=torch.long)
    full[:, 0], full[:, 1:4], full[:, 4] = 2, torch.randint(4, aux.size(), (B, 3)), 3      # BOS w w w EOS pad
    batch.tensors["aux_target_input"] = full[:, :-1].t().contiguous()
    batch.tensors["aux_target_output"] = full[:, 1:].t().contiguous()
    batch.tensors["aux_tgt_lengths"] = torch.full((B,), 4)
    model.train()
    out = model(batch)
    assert torch.isfinite(out["loss"]).all() and out["n_ctc_targets"] == 3 * B          # the EOS is not a CTC label
    out["loss"].backward()
    assert model.ctc_linear.weight.grad.abs().sum() > 0


def test_relative_position_attention_modules_match_the_padded_statement():
    """WavLM's gated bucket bias and Shaw's relative keys, computed on packed rows and handed to the attention op as an
    additive bias, against the textbook padded computation."""
    import math
    import torch.nn.functional as F
    from nmtgminor_b200.models.layers import PackedSeqs
    from nmtgminor_b200.models.speech_encoders import GatedRelPosSelfAttention
    from nmtgminor_b200.models.w2vbert import ShawRelPosSelfAttention
    from nmtgminor_b200.ops.reference import pad_packed, unpad_packed
    torch.manual_seed(0)
    lengths = [9, 4, 6]
    n, T, H, h = sum(lengths), max(lengths), 32, 2
    cu = torch.zeros(4, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    seqs = PackedSeqs(torch.zeros(n, dtype=torch.long), torch.zeros(n, dtype=torch.long), cu, T)
    x = torch.randn(n, H)
    wav = GatedRelPosSelfAttention(H, h, 0.0, num_buckets=16, max_distance=20).eval()
    shaw = ShawRelPosSelfAttention(H, h, 0.0, max_left=4, max_right=2).eval()
    for mod in (wav, shaw):
        with torch.no_grad():
            got = mod(x, seqs)
            qkv, valid = pad_packed(mod.qkv(x), cu, T)
            B = qkv.shape[0]
            q, k, v = (t.view(B, T, h, H // h).transpose(1, 2) for t in qkv.float().split(H, dim=-1))
            if mod is wav:
                gate = mod.grep_linear(q).view(B, h, T, 2, 4).sum(-1)
                ga, gb = torch.sigmoid(gate).chunk(2, dim=-1)
                bias = (ga * (gb * mod.grep_a - 1.0) + 2.0) * mod.position_bias(T, x.device, ("t", 0))[None].float()
                scale = (H // h) ** -0.5
            else:
                scale = (H // h) ** -0.5
                by_offset = torch.matmul(q, mod.rel_k.weight.float().t()) * scale
                bias = by_offset.gather(-1, mod.rel_index(T, x.device)[None, None].expand(B, h, T, T))
            s = torch.matmul(q, k.transpose(-1, -2)) * scale + bias
            s = s.masked_fill(~valid[:, None, None, :], float("-inf"))
            ctx = torch.matmul(torch.softmax(s, -1), v).transpose(1, 2).reshape(B, T, H) * valid.unsqueeze(-1)
            want = mod.out(unpad_packed(ctx, cu, n), dropout_p=0.0, residual=None)
        assert torch.allclose(got, want, atol=1e-5), type(mod).__name__


def test_transducer_branch_of_the_speech_model():
    """-transducer_loss: the RNN-T term is computed from encoder frames and decoder states through the joint, weighted
    and added to the attention loss; blank is the padding id."""
    from nmtgminor_b200.data.dataset import collate
    from nmtgminor_b200.ops.sequence import transducer_loss_reference
    torch.manual_seed(0)
    d = synthetic_dict(30)
    opt = default_options(["-model", "speech_transformer", "-encoder_type", "audio", "-input_size", "8", "-model_size", "32",
                           "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-transducer_loss", "0.5", "-dropout", "0",
                           "-attn_dropout", "0", "-word_dropout", "0", "-emb_dropout", "0"])
    m = build_model(opt, {"tgt": d}).train()
    src = [torch.randn(40, 8), torch.randn(28, 8)]
    tgt = [torch.tensor([2, 11, 12, 13, 3]), torch.tensor([2, 14, 3])]
    b = collate(src, tgt, src_type="audio", padded=True, packed=True)
    out = m(b)
    assert out["transducer_numel"] == 4
    total, nmt, rnnt = float(out["loss"].sum()), float(out["nmt_loss"].sum()), float(out["transducer_loss"])
    assert abs(total - (nmt + 0.5 * rnnt)) < 1e-3 * total
    # the same term from the pieces
    with torch.no_grad():
        context, s = m.encode(b)
        f = s.pad(context, time_first=False).float()
        g = out["tgt"].pad(out["hidden_packed"], time_first=False).float()
        f_len = (s.cu[1:] - s.cu[:-1]).int()
        joint = torch.relu(f[:, :, None, :] + g[:, None, :, :])
        logp = torch.log_softmax(m.transducer_linear(joint), -1)
        labels = torch.tensor([[11, 12, 13], [14, 0, 0]])
        want = transducer_loss_reference(logp, labels, f_len[:2], torch.tensor([3, 1], dtype=torch.int32), 0).sum()
    assert abs(float(want) - rnnt) < 1e-3 * rnnt
    out["loss"].sum().backward()
    assert m.transducer_linear.weight.grad.abs().sum() > 0
    m.eval()
    with torch.no_grad():
        assert "transducer_loss" not in m(b)


def test_language_prediction_heads_of_the_speech_model():
    """-predict_language: frame-level and token-level language heads trained next to the translation loss, and the
    per-utterance prediction used by the language predictor."""
    from nmtgminor_b200.data.dataset import collate
    torch.manual_seed(0)
    d = synthetic_dict(30)
    dicts = {"tgt": d, "langs": {"en": 0, "de": 1, "vi": 2}}
    opt = default_options(["-model", "speech_transformer", "-encoder_type", "audio", "-input_size", "8", "-model_size", "32",
                           "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-predict_language", "1", "-dropout", "0",
                           "-attn_dropout", "0", "-word_dropout", "0", "-emb_dropout", "0"])
    m = build_model(opt, dicts).train()
    assert m.enc_lid.out_features == 3 and m.dec_lid.out_features == 3
    src = [torch.randn(40, 8), torch.randn(28, 8)]
    tgt = [torch.tensor([2, 11, 12, 13, 3]), torch.tensor([2, 14, 3])]
    b = collate(src, tgt, src_type="audio", padded=True, packed=True, src_lang=torch.tensor([0, 2]), tgt_lang=torch.tensor([1, 1]))
    out = m(b)
    assert abs(float(out["loss"].sum()) - float(out["nmt_loss"].sum()) - 0.01 * float(out["lid_loss"])) < 1e-3
    # every encoder frame of utterance 0 is labelled 0 and of utterance 1 is labelled 2; six decoder positions labelled 1
    n_frames = int(out["src"].cu[-1])
    uniform = (n_frames + 6) * math.log(3)
    assert 0.3 * uniform < float(out["lid_loss"]) < 3 * uniform
    out["loss"].sum().backward()
    assert m.enc_lid.weight.grad.abs().sum() > 0 and m.dec_lid.weight.grad.abs().sum() > 0
    opt_sgd = torch.optim.SGD(list(m.enc_lid.parameters()), lr=0.5)
    for _ in range(60):
        opt_sgd.zero_grad()
        m(b)["loss"].sum().backward()
        opt_sgd.step()
    m.eval()
    pred = m.predict_language(b)
    assert pred.shape == (2, 3) and pred.argmax(-1).tolist() == [0, 2]


def test_relative_self_attention_bias_operand_path_matches_padded_path():
    """Sequences that do not fit the one-tile relative kernel go through the packed attention kernels with the position
    term and the content bias as one additive operand; on CPU the same routing runs on the PyTorch statement."""
    import torch
    from nmtgminor_b200.models.layers import PackedSeqs
    from nmtgminor_b200.models.relative_transformer import RelativeSelfAttention
    torch.manual_seed(3)
    for causal in (False, True):
        m = RelativeSelfAttention(32, 2, 0.0, causal).eval()
        with torch.no_grad():
            m.r_w_bias.normal_(0, 0.3)
            m.r_r_bias.normal_(0, 0.3)
        lengths = [9, 4, 6]
        n = sum(lengths)
        cu = torch.zeros(4, dtype=torch.int32)
        cu[1:] = torch.tensor(lengths).cumsum(0)
        seqs = PackedSeqs(torch.zeros(n, dtype=torch.long), torch.zeros(n, dtype=torch.long), cu, max(lengths))
        x = torch.randn(n, 32, requires_grad=True)
        a = m(x, seqs)
        ga = torch.autograd.grad(a.square().sum(), [x] + list(m.parameters()), allow_unused=True)
        m.force_bias_path = True
        b = m(x, seqs)
        gb = torch.autograd.grad(b.square().sum(), [x] + list(m.parameters()), allow_unused=True)
        assert torch.allclose(a, b, atol=1e-5)
        for u, v in zip(ga, gb):
            assert (u is None) == (v is None)
            if u is not None:
                assert torch.allclose(u, v, atol=1e-4, rtol=1e-4)


def test_language_adapters_in_the_speech_encoder_and_the_pretrained_decoder(dicts, tmp_path):
    """``-wav2vec_adapter 1 -decoder_adapter 1``: one adapter per language and layer; a batch trains the adapters of its
    own source / target language only, and decoding takes the same path."""
    torch.manual_seed(5)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=2, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    argv = ["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50",
            "-wav2vec_adapter", "1", "-decoder_adapter", "1"]
    model = build_model(default_options(argv + COMMON), dicts)
    assert len(model.encoder.adapters) == 2 and len(model.encoder.adapters[0].adapters) == 2
    assert len(model.decoder.adapters) == 2 and len(model.decoder.adapters[0].adapters) == 2
    batch = synthetic_audio_batch(2, 120, "wav", 3000, 6000)
    with pytest.raises(ValueError, match="language"):
        model(batch)
    batch.tensors["source_lang"] = torch.tensor([0])
    batch.tensors["target_lang"] = torch.tensor([1])
    # the up-projection starts at zero (identity adapter): move it so that the adapters matter
    with torch.no_grad():
        for stack in (model.encoder.adapters, model.decoder.adapters):
            for per_layer in stack:
                for a in per_layer.adapters:
                    a.up.weight.normal_(0, 0.05)
    out = model(batch)
    out["loss"].backward()

    def touched(adapter):
        return adapter.up.weight.grad is not None and float(adapter.up.weight.grad.abs().sum()) > 0
    assert touched(model.encoder.adapters[0].adapters[0]) and not touched(model.encoder.adapters[0].adapters[1])
    assert touched(model.decoder.adapters[1].adapters[1]) and not touched(model.decoder.adapters[1].adapters[0])
    # another target language gives another loss; decoding runs through the adapters too
    model.eval()
    with torch.no_grad():
        a = float(model(batch)["loss"])
        batch.tensors["target_lang"] = torch.tensor([0])
        b = float(model(batch)["loss"])
    assert abs(a - b) > 1e-6
    hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=4))
    assert len(hyps) == 2


def test_ctc_loss_delay_switches_the_term_on_after_the_given_number_of_updates(dicts, tmp_path):
    torch.manual_seed(6)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    argv = ["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50",
            "-ctc_loss", "0.3", "-ctc_loss_delay", "2"]
    model = build_model(default_options(argv + COMMON), dicts)
    batch = synthetic_audio_batch(2, 120, "wav", 3000, 6000)
    for step, expected in ((0, False), (2, False), (3, True)):
        model.num_updates = step
        out = model(batch)
        assert ("ctc_loss" in out) == expected, step


def test_stochastic_sublayer_tosses_one_coin_per_sublayer(dicts):
    """With ``-stochastic_sublayer`` a layer can keep its attention and drop its feed-forward block (or the other way
    round); without it the layer is kept or dropped as a whole."""
    from nmtgminor_b200.models.layers import EncoderLayer
    torch.manual_seed(0)
    model = build_model(default_options(["-model", "transformer", "-death_rate", "0.5", "-stochastic_sublayer"] + COMMON), dicts)
    layers = [m for m in model.modules() if isinstance(m, EncoderLayer)]
    assert layers and all(l.stochastic_sublayer for l in layers)
    layer = layers[-1]
    layer.death_rate = 0.5
    layer.train()
    calls = {"attn": 0, "ffn": 0}
    layer.attn.register_forward_hook(lambda *a: calls.__setitem__("attn", calls["attn"] + 1))
    layer.ffn.register_forward_hook(lambda *a: calls.__setitem__("ffn", calls["ffn"] + 1))
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    seqs = batch.packed_source()
    x = torch.randn(seqs.tokens.shape[0], layer.attn_norm.weight.shape[0])
    patterns = set()
    for _ in range(40):
        before = dict(calls)
        layer(x, seqs)
        patterns.add((calls["attn"] - before["attn"], calls["ffn"] - before["ffn"]))
    assert {(1, 0), (0, 1)} & patterns, patterns          # mixed patterns occur
    layer.stochastic_sublayer = False
    patterns = set()
    for _ in range(40):
        before = dict(calls)
        layer(x, seqs)
        patterns.add((calls["attn"] - before["attn"], calls["ffn"] - before["ffn"]))
    assert patterns <= {(0, 0), (1, 1)}, patterns


def test_rotary_positions_make_attention_depend_on_distance_only(dicts, tmp_path):
    from nmtgminor_b200.models.layers import PackedSeqs, SelfAttention, rotate_queries_and_keys
    torch.manual_seed(7)
    heads, d, n = 2, 8, 6
    qkv = torch.randn(n, 3 * heads * d)
    a = rotate_queries_and_keys(qkv, torch.arange(n), heads).view(n, 3, heads, d)
    b = rotate_queries_and_keys(qkv, torch.arange(n) + 11, heads).view(n, 3, heads, d)
    sa = torch.einsum("ihd,jhd->hij", a[:, 0], a[:, 1])
    sb = torch.einsum("ihd,jhd->hij", b[:, 0], b[:, 1])
    assert torch.allclose(sa, sb, atol=1e-4)                       # a common shift changes no score
    assert torch.equal(a[:, 2], qkv.view(n, 3, heads, d)[:, 2])    # values untouched
    plain = torch.einsum("ihd,jhd->hij", qkv.view(n, 3, heads, d)[:, 0], qkv.view(n, 3, heads, d)[:, 1])
    assert not torch.allclose(sa, plain, atol=1e-3)
    # the module: with rotary on, the output changes and still backpropagates
    att = SelfAttention(16, 2).eval()
    cu = torch.tensor([0, 4, 6], dtype=torch.int32)
    seqs = PackedSeqs(torch.ones(6, dtype=torch.long), torch.tensor([0, 1, 2, 3, 0, 1]), cu, 4)
    x = torch.randn(6, 16, requires_grad=True)
    y0 = att(x, seqs)
    att.rotary = True
    y1 = att(x, seqs)
    assert not torch.allclose(y0, y1, atol=1e-4)
    y1.sum().backward()
    assert x.grad is not None
    # the flag reaches the wav2vec 2.0 encoder layers
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    model = build_model(default_options(["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model",
                                         "mbart50", "-rotary_position_encoding"] + COMMON), dicts)
    assert all(l.attn.rotary for l in model.encoder.layers)
    out = model(synthetic_audio_batch(2, 120, "wav", 3000, 6000))
    assert torch.isfinite(out["loss"]).all()


def test_weight_drop_and_factorised_weight_options(dicts):
    """``-weight_drop`` masks the feed-forward weights in training only; ``-mfw_multiplicative`` / ``-mfw_activation`` change
    the per-language weight as the formula says."""
    from nmtgminor_b200.models.layers import FeedForward
    from nmtgminor_b200.models.multilingual import FactorizedLinear
    torch.manual_seed(8)
    model = build_model(default_options(["-model", "transformer", "-weight_drop", "0.5"] + COMMON), dicts)
    ffns = [m for m in model.modules() if isinstance(m, FeedForward)]
    assert ffns and all(f.weight_drop == 0.5 for f in ffns)
    f = ffns[0]
    f.dropout = 0.0
    x = torch.randn(5, f.fc1.weight.shape[1])
    f.eval()
    assert torch.allclose(f(x), f(x))
    f.train()
    a, b = f(x), f(x)
    assert not torch.allclose(a, b)                        # two different weight masks
    a.sum().backward()
    assert f.fc1.weight.grad is not None and float((f.fc1.weight.grad == 0).float().mean()) > 0.2   # dropped entries get no gradient
    lin = FactorizedLinear(6, 4, n_languages=2, rank=1, multiplicative=True, activation="silu").eval()
    with torch.no_grad():
        lin.rm.uniform_(0.5, 1.5)
        lin.sm.uniform_(0.5, 1.5)
    want = torch.nn.functional.silu(lin.weight * (lin.rm[1].t() @ lin.sm[1])) + lin.r[1].t() @ lin.s[1]
    assert torch.allclose(lin.weight_for(1), want, atol=1e-6)
    ml = build_model(default_options(["-model", "multilingual_translator", "-multilingual_factorized_weights", "-mfw_multiplicative",
                                      "-mfw_activation", "gelu"] + COMMON), dicts)
    fl = [m for m in ml.modules() if isinstance(m, FactorizedLinear)]
    assert fl and all(m.multiplicative and m.activation == "gelu" for m in fl)


def test_relative_attention_inside_the_wav2vec_encoder(dicts, tmp_path):
    from nmtgminor_b200.models.relative_transformer import RelativeSelfAttention
    torch.manual_seed(9)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    model = build_model(default_options(["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model",
                                         "mbart50", "-wav2vec2_relative_attention"] + COMMON), dicts)
    assert all(isinstance(l.attn, RelativeSelfAttention) for l in model.encoder.layers)
    out = model(synthetic_audio_batch(2, 120, "wav", 3000, 6000))
    out["loss"].backward()
    assert model.encoder.layers[0].attn.r_r_bias.grad is not None


def test_partitioned_multilingual_weights(dicts):
    """``-multilingual_partitioned_weights``: every projection is a per-language mixture of shared matrices, mixed by one
    factor table that all layers share; a batch trains its own language's factor row only."""
    from nmtgminor_b200.models.multilingual import PartitionedLinear
    torch.manual_seed(10)
    model = build_model(default_options(["-model", "multilingual_translator", "-multilingual_partitioned_weights", "-mpw_factor_size", "3"]
                                        + COMMON), dicts)
    lins = [m for m in model.modules() if isinstance(m, PartitionedLinear)]
    assert lins and all(m._factors is model.factor_embeddings for m in lins)
    assert model.factor_embeddings.weight.shape == (2, 3)
    assert sum(1 for n, _ in model.named_parameters() if "factor_embeddings" in n) == 1       # registered once
    lin = lins[0]
    want = sum(model.factor_embeddings.weight[1, f] * lin.shared_weight[:, f] for f in range(3)).view(lin.d_out, lin.d_in)
    assert torch.allclose(lin.weight_for(1), want, atol=1e-6)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    batch.tensors["source_lang"] = torch.tensor([0])
    batch.tensors["target_lang"] = torch.tensor([0])
    out = model(batch)
    out["loss"].backward()
    g = model.factor_embeddings.weight.grad
    assert g is not None and float(g[0].abs().sum()) > 0 and float(g[1].abs().sum()) == 0
    model.eval()
    hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=4))
    assert len(hyps) == batch.size


@pytest.mark.parametrize("extra", [["-multilingual_adapter", "-adapter_bottleneck_size", "16"],
                                   ["-multilingual_factorized_weights", "-mfw_rank", "2"],
                                   ["-multilingual_partitioned_weights", "-mpw_factor_size", "3"]])
def test_multilingual_decoding_matches_the_training_forward(dicts, extra):
    """Step-by-step decoding of the multilingual model gives the distributions of the teacher-forced forward pass: the
    language embedding, per-language weights and adapters all take part in decoding."""
    torch.manual_seed(12)
    model = build_model(default_options(["-model", "multilingual_translator"] + extra + COMMON), dicts).eval()
    with torch.no_grad():
        for m in model.modules():                      # adapters start as the identity: move them so that they matter
            if hasattr(m, "up") and hasattr(m, "down"):
                m.up.weight.normal_(0, 0.1)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    batch.tensors["source_lang"] = torch.tensor([0])
    batch.tensors["target_lang"] = torch.tensor([1])
    with torch.no_grad():
        out = model(batch, return_logits=True)
        want = torch.log_softmax(out["logprobs"].float(), -1)          # [T, B, V]
        tgt_in = batch.get("target_input")                              # [T, B]
        lengths = batch.get("tgt_lengths")
        state = model.create_decoder_state(batch, 1)
        for t in range(min(4, tgt_in.shape[0])):
            lp = model.step(tgt_in[:t + 1].t().contiguous(), state)["log_prob"]     # [B, V]
            rows = (lengths > t).nonzero().squeeze(1) if lengths is not None else torch.arange(lp.shape[0])
            assert torch.allclose(lp[rows], want[t][rows], atol=2e-4), (t, float((lp[rows] - want[t][rows]).abs().max()))


def test_small_structure_switches(dicts):
    """``-no_batch_norm`` / ``-no_input_scale`` on the filterbank encoder, ``-encoder_early_emb_scale`` /
    ``-decoder_late_emb_scale`` on the multilingual model."""
    import math
    import torch.nn as nn
    args = ["-model", "speech_transformer", "-input_size", "40", "-cnn_downsampling"]
    a = build_model(default_options(args + COMMON), dicts)
    b = build_model(default_options(args + ["-no_batch_norm", "-no_input_scale"] + COMMON), dicts)
    assert any(isinstance(m, nn.BatchNorm2d) for m in a.encoder.conv) and not any(isinstance(m, nn.BatchNorm2d) for m in b.encoder.conv)
    assert a.encoder.input_scale == math.sqrt(a.encoder.dim) and b.encoder.input_scale == 1.0
    out = b(synthetic_audio_batch(2, 120, "feats", 40, 80, n_feats=40))
    assert torch.isfinite(out["loss"]).all()
    m0 = build_model(default_options(["-model", "multilingual_translator"] + COMMON), dicts)
    m1 = build_model(default_options(["-model", "multilingual_translator", "-encoder_early_emb_scale", "-decoder_late_emb_scale"] + COMMON), dicts)
    d = m0.lang_embed.embedding_dim
    assert (m0.enc_lang_scale, m0.dec_lang_scale) == (math.sqrt(d), 1.0)
    assert (m1.enc_lang_scale, m1.dec_lang_scale) == (1.0, math.sqrt(d))


def test_wav2vec_channel_masking(dicts, tmp_path):
    """``-wav2vec_spec_augment``: spans of feature channels are zeroed in training and left alone in evaluation."""
    torch.manual_seed(14)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=512, encoder_layers=1, encoder_attention_heads=8, encoder_ffn_embed_dim=128)
    dec = _cfg(tmp_path, "dec.json", d_model=64, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=120, pad_token_id=0)
    model = build_model(default_options(["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model",
                                         "mbart50", "-wav2vec_spec_augment"] + COMMON), dicts)
    assert model.encoder.mask_channel_prob == 0.2 and model.encoder.mask_channel_length == 64
    batch = synthetic_audio_batch(2, 120, "wav", 3000, 6000)
    seen = {}
    model.encoder.pos_conv.register_forward_hook(lambda mod, inp, out: seen.__setitem__("x", inp[0].detach()))
    model.train()
    model(batch)
    zero_cols = (seen["x"].abs().sum(1) == 0).sum(-1)                  # per utterance: channels that are zero at every frame
    assert int(zero_cols.max()) >= 1
    model.eval()
    with torch.no_grad():
        model(batch)
    assert int((seen["x"].abs().sum(1) == 0).sum()) == 0


def test_no_ffn_and_depthwise_conv_change_the_encoder_layers_and_survive_a_checkpoint(dicts):
    from nmtgminor_b200.models.layers import EncoderLayer, PackedConvolution
    from nmtgminor_b200.train.checkpoint import load_model_state, model_state_for_saving
    torch.manual_seed(0)
    flags = ["-model", "transformer", "-depthwise_conv", "-conv_kernel", "5", "-no_ffn", "-macaron"] + COMMON
    model = build_model(default_options(flags), dicts)
    enc_layers = [m for m in model.encoder.modules() if isinstance(m, EncoderLayer)]
    assert enc_layers and all(isinstance(m.conv, PackedConvolution) and m.ffn is None for m in enc_layers)
    assert not any(".ffn." in k for k in model.encoder.state_dict()) and any(".ffn." in k for k in model.decoder.state_dict())
    from nmtgminor_b200.models.layers import PackedSeqs
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    out = model(batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and enc_layers[0].conv.dw.weight.grad.abs().sum() > 0
    # a sentence's encoding does not depend on what it is batched with (the convolution never reads across sequences)
    model.eval()
    with torch.no_grad():
        src = batch.packed_source()
        full = model.encoder(src)
        n0 = int(src.cu[1])
        first = PackedSeqs(src.tokens[:n0], src.positions[:n0], src.cu[:2], n0)
        assert torch.allclose(model.encoder(first), full[:n0], atol=1e-5)
    # structure switches add parameters; all of them come back from a saved state (also the macaron block and the gates)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    saved = model_state_for_saving(model)
    fresh = build_model(default_options(flags), dicts)
    missing, unexpected = load_model_state(fresh, saved)
    assert not missing and not unexpected
    assert all(torch.allclose(a, b) for a, b in zip(model.state_dict().values(), fresh.state_dict().values()))
    gated = build_model(default_options(["-model", "transformer", "-rezero"] + COMMON), dicts)
    with torch.no_grad():
        for m in gated.modules():
            if hasattr(m, "gates"):
                m.gates.fill_(0.3)
    again = build_model(default_options(["-model", "transformer", "-rezero"] + COMMON), dicts)
    assert load_model_state(again, model_state_for_saving(gated))[0] == []
    assert float(again.encoder.layers[0].gates[0]) == pytest.approx(0.3)
    with pytest.raises(NotImplementedError, match="no_ffn"):
        build_model(default_options(["-model", "LSTM", "-no_ffn"] + COMMON), dicts)


def test_per_language_output_projection_and_absolute_positions(dicts):
    torch.manual_seed(0)
    flags = ["-model", "speech_transformer", "-input_size", "40", "-multilingual_linear_projection"] + COMMON
    model = build_model(default_options(flags), dicts).eval()
    assert model.encoder.linear_proj.shape == (2, 64, 64)
    batch = synthetic_audio_batch(3, 120, "feats", 40, 80, n_feats=40)
    batch.tensors["source_lang"] = torch.tensor([1])
    batch.tensors["target_lang"] = torch.tensor([0])
    with torch.no_grad():
        ctx1, _ = model.encode(batch)
        model.encoder.linear_proj[1].copy_(torch.eye(64))
        plain, _ = model.encode(batch)
        model.encoder.linear_proj[1].mul_(2.0)
        doubled, _ = model.encode(batch)
        model.encoder.linear_proj[0].zero_()                      # another language's matrix is not read
        assert torch.allclose(model.encode(batch)[0], doubled)
    assert torch.allclose(doubled, 2 * plain, atol=1e-5) and not torch.allclose(ctx1, plain)
    model.train()
    model(batch)["loss"].backward()
    g = model.encoder.linear_proj.grad
    assert g[1].abs().sum() > 0 and g[0].abs().sum() == 0
    # absolute positions on top of relative attention: the embedding now adds the sinusoidal table
    rel = build_model(default_options(["-model", "relative_transformer"] + COMMON), dicts).eval()
    both = build_model(default_options(["-model", "relative_transformer", "-absolute_position_encoding"] + COMMON), dicts).eval()
    both.load_state_dict(rel.state_dict(), strict=False)
    text = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    with torch.no_grad():
        a, b = rel.encode(text)[0], both.encode(text)[0]
    assert a.shape == b.shape and not torch.allclose(a, b, atol=1e-3)


def test_favor_attention_estimates_softmax_attention_in_the_encoder(dicts):
    """``-favor_attention``: with many random features the encoder output approaches the exact-attention output, and
    it does not depend on the padding of the batch."""
    from nmtgminor_b200.models.layers import PackedSeqs, SelfAttention
    torch.manual_seed(0)
    exact = build_model(default_options(["-model", "transformer"] + COMMON), dicts).eval()
    favor = build_model(default_options(["-model", "transformer", "-favor_attention"] + COMMON), dicts).eval()
    favor.load_state_dict(exact.state_dict(), strict=False)
    attn = [m for m in favor.encoder.modules() if isinstance(m, SelfAttention)]
    assert attn and all(m.favor_projection is not None for m in attn)
    assert all(m.favor_projection is None for m in favor.decoder.modules() if isinstance(m, SelfAttention))
    for i, m in enumerate(attn):
        m.enable_favor(nb_features=4096, seed=i)
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    with torch.no_grad():
        src = batch.packed_source()
        a, b = exact.encoder(src), favor.encoder(src)
        n0 = int(src.cu[1])
        alone = favor.encoder(PackedSeqs(src.tokens[:n0], src.positions[:n0], src.cu[:2], n0))
    assert float((a - b).abs().mean()) < 0.1 * float(a.abs().mean())
    assert torch.allclose(alone, b[:n0], atol=1e-4)
    favor.train()
    out = favor(batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and attn[0].qkv.weight.grad.abs().sum() > 0
    with pytest.raises(NotImplementedError, match="favor_attention"):
        build_model(default_options(["-model", "LSTM", "-favor_attention"] + COMMON), dicts)


def test_no_decoder_builds_a_ctc_only_speech_model_that_learns_and_decodes(dicts, tmp_path):
    from nmtgminor_b200.models.pretrained import SpeechCTCModel
    torch.manual_seed(0)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    model = build_model(default_options(["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-no_decoder"] + COMMON), dicts)
    assert isinstance(model, SpeechCTCModel) and model.decoder is None
    assert not any(k.startswith("decoder") or k.startswith("generator") for k in model.state_dict())
    batch = synthetic_audio_batch(2, 120, "wav", 3000, 4000, tgt_min=3, tgt_max=5)
    opt = torch.optim.Adam(model.parameters(), lr=2e-3)
    model.train()
    first = None
    for _ in range(60):
        opt.zero_grad()
        out = model(batch)
        out["loss"].backward()
        opt.step()
        first = first if first is not None else float(out["loss"])
    assert float(out["loss"]) < 0.2 * first
    model.eval()
    hyps = model.ctc_greedy(batch)
    gold = batch.get("target_output").t()
    for (tokens, score), row in zip(hyps, gold):
        assert tokens == [int(t) for t in row if int(t) not in (0, 3)] and score <= 0
    with pytest.raises(NotImplementedError, match="no_decoder"):
        build_model(default_options(["-model", "transformer", "-no_decoder"] + COMMON), dicts)
    # the translator takes the best path instead of searching
    from nmtgminor_b200.inference.translator import Translator
    tr = Translator.__new__(Translator)
    tr.model, tr.cuda, tr.cfg = model, False, None
    out = tr.translate_batch(batch)
    assert [h[0].tokens for h in out] == [t for t, _ in hyps]


def test_branchformer_layers_add_a_cgmlp_branch(dicts, tmp_path):
    from nmtgminor_b200.models.layers import ConvolutionalGatingMLP, EncoderLayer, PackedSeqs
    torch.manual_seed(0)
    enc = _cfg(tmp_path, "enc.json", encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)
    model = build_model(default_options(["-model", "wav2vec2_transformer", "-enc_config_file", enc, "-branchformer", "-conv_kernel", "7"]
                                        + COMMON), dicts)
    layers = [m for m in model.encoder.modules() if isinstance(m, EncoderLayer)]
    assert len(layers) == 2 and all(isinstance(m.cgmlp, ConvolutionalGatingMLP) and m.merge_proj.in_features == 128 for m in layers)
    batch = synthetic_audio_batch(2, 120, "wav", 3000, 6000)
    out = model(batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"])
    for name in ("cgmlp.proj1.weight", "cgmlp.gate_conv.weight", "merge_conv.weight", "merge_proj.weight", "attn.qkv.weight"):
        g = dict(layers[0].named_parameters())[name].grad
        assert g is not None and g.abs().sum() > 0, name
    # at initialisation the gate is GELU(1): the cgMLP output is proj2(r * GELU(1)); and sequences do not mix
    layer = layers[0].eval()
    seqs = PackedSeqs(torch.zeros(9, dtype=torch.long), torch.arange(9) % 5, torch.tensor([0, 5, 9], dtype=torch.int32), 5)
    x = torch.randn(9, 64)
    with torch.no_grad():
        r, _ = torch.nn.functional.gelu(layer.cgmlp.proj1(x)).chunk(2, -1)
        expect = layer.cgmlp.proj2(r * torch.nn.functional.gelu(torch.ones(())))
        assert torch.allclose(layer.cgmlp(x, seqs), expect, atol=1e-4)
        both = layer(x, seqs)
        first = layer(x[:5], PackedSeqs(seqs.tokens[:5], seqs.positions[:5], seqs.cu[:2], 5))
    assert torch.allclose(both[:5], first, atol=1e-5)
    with pytest.raises(NotImplementedError, match="branchformer"):
        build_model(default_options(["-model", "LSTM", "-branchformer"] + COMMON), dicts)


@pytest.mark.parametrize("kind", ["maxout", "linear_swish_linear"])
def test_activation_layer_variants_of_the_xl_language_model(dicts, kind):
    from nmtgminor_b200.models.relative_transformer import MaxOutFeedForward
    torch.manual_seed(0)
    lm = build_model(default_options(["-model", "transformer_xl_lm", "-activation_layer", kind] + COMMON), dicts)
    ffn = lm.decoder.layers[0].ffn
    if kind == "maxout":
        assert isinstance(ffn, MaxOutFeedForward) and ffn.maxout.pool == 2 and ffn.maxout.lin.out_features == 128
        x = torch.randn(5, 64)
        cand = ffn.maxout.lin(x).view(5, 64, 2)
        assert torch.allclose(ffn(x), cand.max(-1).values)
    else:
        assert ffn.activation == "silu"
    batch = token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]
    out = lm(batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and all(p.grad is not None for p in ffn.parameters())
    with pytest.raises(NotImplementedError, match="activation_layer"):
        build_model(default_options(["-model", "transformer", "-activation_layer", kind] + COMMON), dicts)

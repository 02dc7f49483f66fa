"""Pretrained weights and reference-named state dicts: the reference's own modules (from ``baseline/_ref``, random
weights, CPU fp32) are the oracle.  Their state dicts are written to disk, loaded through the command-line options of
this framework (``-dec_state_dict`` ...), and the two forward passes must agree; the way back (this framework's
checkpoint naming into the reference module) is checked too.  Skipped when the reference is not installed."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _reference():
    from bench_reference import import_reference, make_opt, reference_available
    ok, why = reference_available()
    if not ok:
        pytest.skip(why)
    onmt, options = import_reference()
    return onmt, options, make_opt


def _packed(ids):
    from nmtgminor_b200.models.layers import PackedSeqs
    B, T = ids.shape
    return PackedSeqs.from_padded(ids, torch.full((B,), T))


def _reference_mbart_decoder(dim=64, heads=2, layers=2, ffn=128, vocab=300):
    onmt, options, make_opt = _reference()
    from pretrain_module.configuration_mbart import MBartConfig
    from pretrain_module.modeling_mbart import MBartDecoder
    opt = make_opt(options, ["-data", "none", "-model", "wav2vec2_bert", "-dropout", "0.0", "-attn_dropout", "0.0", "-word_dropout", "0.0"])
    cfg = MBartConfig(vocab_size=vocab, d_model=dim, decoder_layers=layers, decoder_attention_heads=heads, decoder_ffn_dim=ffn,
                      encoder_layers=layers, encoder_attention_heads=heads, encoder_ffn_dim=ffn, max_position_embeddings=64,
                      pad_token_id=1, scale_embedding=True, dropout=0.0)
    torch.manual_seed(0)
    dec = MBartDecoder(cfg, opt).eval()
    with torch.no_grad():                       # biases and LayerNorms away from their trivial initial values
        for n, p in dec.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    hf_names = {k: v.clone() for k, v in dec.state_dict().items()}
    for m in dec.modules():                     # what the reference's optimize_model does before training
        if hasattr(m, "convert_fast_attention"):
            m.convert_fast_attention()
    return dec, hf_names, {k: v.clone() for k, v in dec.state_dict().items()}


def _our_mbart_model(tmp_path, extra):
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import default_options
    import json
    cfg = tmp_path / "dec.json"
    cfg.write_text(json.dumps(dict(d_model=64, decoder_layers=2, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=300,
                                   max_position_embeddings=64, pad_token_id=1)))
    d = synthetic_dict(300)
    opt = default_options(["-model", "pretrain_transformer", "-enc_pretrained_model", "mbart50", "-dec_pretrained_model", "mbart50",
                           "-dec_config_file", str(cfg), "-model_size", "64", "-layers", "2", "-n_heads", "2", "-inner_size", "128",
                           "-dropout", "0.0", "-attn_dropout", "0.0"] + extra)
    return build_model(opt, {"src": d, "tgt": d}).eval()


@pytest.mark.parametrize("layout", ["module_names", "fast_layout"])
def test_mbart_decoder_state_dict_loads_through_the_option_and_matches_the_reference(tmp_path, layout):
    ref, hf_names, fast = _reference_mbart_decoder()
    path = tmp_path / "dec_state.pt"
    torch.save(hf_names if layout == "module_names" else fast, path)
    model = _our_mbart_model(tmp_path, ["-dec_state_dict", str(path)])
    torch.manual_seed(1)
    B, T, S = 3, 7, 9
    ids = torch.randint(4, 300, (B, T))
    enc = torch.randn(S, B, 64)
    with torch.no_grad():
        want = ref(input_ids=ids, attention_mask=torch.zeros(B, T, dtype=torch.bool), encoder_hidden_states=enc,
                   encoder_attention_mask=torch.zeros(B, S, dtype=torch.bool))[0]          # [T, B, H]
        tgt = _packed(ids)
        mem_seqs = _packed(torch.ones(B, S, dtype=torch.long))
        memory = enc.transpose(0, 1).reshape(B * S, 64)
        got = model.decoder(tgt, memory, mem_seqs).view(B, T, 64).transpose(0, 1)
    assert (got - want).abs().max().item() < 1e-4, (got - want).abs().max().item()


def test_checkpoint_naming_round_trips_into_the_reference_decoder(tmp_path):
    """A checkpoint of this framework (reference naming, fused layout) restores the reference's converted module."""
    from nmtgminor_b200.train.checkpoint import model_state_for_saving
    ref, _hf, fast = _reference_mbart_decoder()
    model = _our_mbart_model(tmp_path, [])
    saved = model_state_for_saving(model)
    dec_part = {k[len("decoder."):]: v for k, v in saved.items() if k.startswith("decoder.")}
    assert set(fast.keys()) <= set(dec_part.keys()), sorted(set(fast) - set(dec_part))[:5]
    ref.load_state_dict({k: dec_part[k] for k in fast}, strict=True)
    B, T, S = 2, 5, 6
    ids = torch.randint(4, 300, (B, T))
    enc = torch.randn(S, B, 64)
    with torch.no_grad():
        want = ref(input_ids=ids, attention_mask=torch.zeros(B, T, dtype=torch.bool), encoder_hidden_states=enc,
                   encoder_attention_mask=torch.zeros(B, S, dtype=torch.bool))[0]
        got = model.decoder(_packed(ids), enc.transpose(0, 1).reshape(B * S, 64), _packed(torch.ones(B, S, dtype=torch.long)))
        got = got.view(B, T, 64).transpose(0, 1)
    assert (got - want).abs().max().item() < 1e-4


def test_whisper_checkpoint_loads_and_matches_the_hugging_face_model(tmp_path):
    """The reference's Whisper path trains Hugging Face's ``WhisperForConditionalGeneration`` (its model class derives
    from it), so that class with random weights is the oracle: its state dict, loaded through ``load_whisper_state``,
    must reproduce encoder states and decoder states."""
    transformers = pytest.importorskip("transformers")
    import json
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.models.pretrained_io import load_whisper_state
    from nmtgminor_b200.options import default_options
    cfg = transformers.WhisperConfig(vocab_size=300, num_mel_bins=80, d_model=64, encoder_layers=2, decoder_layers=2,
                                     encoder_attention_heads=2, decoder_attention_heads=2, encoder_ffn_dim=128, decoder_ffn_dim=128,
                                     max_source_positions=50, max_target_positions=32, dropout=0.0, attention_dropout=0.0,
                                     activation_dropout=0.0, pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = transformers.WhisperForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1 and "embed_positions" not in n:
                p.add_(torch.randn_like(p) * 0.1)
    jf = tmp_path / "whisper.json"
    jf.write_text(json.dumps(dict(d_model=64, encoder_layers=2, decoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=128,
                                  num_mel_bins=80, max_source_positions=50, max_target_positions=32, vocab_size=300, pad_token_id=0)))
    d = synthetic_dict(300)
    opt = default_options(["-model", "whisper", "-dec_config_file", str(jf), "-model_size", "64", "-n_heads", "2", "-inner_size", "128",
                           "-layers", "2", "-dropout", "0.0", "-attn_dropout", "0.0"])
    model = build_model(opt, {"src": d, "tgt": d}).eval()
    load_whisper_state(model, hf.state_dict(), verbose=False)
    B, frames, T = 2, 100, 6
    feats = torch.randn(B, 80, frames)
    ids = torch.randint(3, 300, (B, T))
    with torch.no_grad():
        enc_want = hf.model.encoder(feats).last_hidden_state                              # [B, 50, 64]
        dec_want = hf.model.decoder(input_ids=ids, encoder_hidden_states=enc_want).last_hidden_state
        src = torch.cat([torch.ones(frames, B, 1), feats.permute(2, 0, 1)], dim=-1)      # [T, B, 1 + mels], channel 0 = real frame
        context, src_seqs = model.encoder(src)
        enc_got = context.view(B, -1, 64)
        dec_got = model.decoder(_packed(ids), context, src_seqs).view(B, T, 64)
    assert (enc_got - enc_want).abs().max().item() < 2e-4, (enc_got - enc_want).abs().max().item()
    assert (dec_got - dec_want).abs().max().item() < 2e-4, (dec_got - dec_want).abs().max().item()


def test_fairseq_named_wav2vec2_checkpoint_loads_through_the_option(tmp_path):
    """The reference's wav2vec 2.0 classes cannot be imported here (they need ``omegaconf``), so the oracle is this
    framework's own encoder: its weights are written under fairseq's names (separate q / k / v projections,
    ``weight_g`` / ``weight_v`` of the positional convolution, ``feature_extractor.conv_layers.i.0`` ...) inside a
    ``{'cfg': {'model': ...}, 'model': ...}`` file, and a fresh model given ``-wav2vec2_pretrained_model <file>`` must
    compute the same encoder states."""
    import json
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.models import pretrained_io as io
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import default_options
    enc_cfg = tmp_path / "enc.json"
    enc_cfg.write_text(json.dumps(dict(encoder_embed_dim=64, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_embed_dim=128)))
    dec_cfg = tmp_path / "dec.json"
    dec_cfg.write_text(json.dumps(dict(d_model=64, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=128, vocab_size=300,
                                       pad_token_id=1)))
    d = synthetic_dict(300)
    args = ["-model", "wav2vec2_bert", "-enc_config_file", str(enc_cfg), "-dec_config_file", str(dec_cfg), "-dec_pretrained_model", "mbart50",
            "-model_size", "64", "-n_heads", "2", "-inner_size", "128", "-layers", "1", "-dropout", "0.0", "-attn_dropout", "0.0"]
    torch.manual_seed(0)
    donor = build_model(default_options(args), {"src": d, "tgt": d}).eval()
    heads = 2
    fast = io.wav2vec2_to_reference({k: v.clone() for k, v in donor.encoder.state_dict().items()}, heads)
    fairseq = {}
    for k, v in fast.items():                    # fast layout -> the separate projections a fairseq file has
        if k.endswith("self_attn.proj_weight") or k.endswith("self_attn.proj_bias"):
            q, kk, vv = io.deinterleave(v, heads, 3).chunk(3, 0)
            base, what = k.rsplit(".proj_", 1)
            for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                fairseq["%s.%s.%s" % (base, name, what)] = t.clone()
        else:
            fairseq[k] = v
    fairseq["quantizer.vars"] = torch.zeros(1, 4, 8)          # pre-training heads that a real file carries and nobody needs
    fairseq["final_proj.weight"] = torch.zeros(8, 64)
    path = tmp_path / "wav2vec_small.pt"
    torch.save({"cfg": {"model": {"encoder_embed_dim": 64, "encoder_layers": 2}}, "model": fairseq}, path)
    assert io.wav2vec2_config_from_checkpoint(str(path))["encoder_layers"] == 2
    torch.manual_seed(7)
    model = build_model(default_options(args + ["-wav2vec2_pretrained_model", str(path)]), {"src": d, "tgt": d}).eval()
    wav = torch.randn(4000, 2, 1)
    src = torch.cat([torch.ones(4000, 2, 1), wav], dim=-1)
    with torch.no_grad():
        want, _ = donor.encoder(src)
        got, _ = model.encoder(src)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max().item()
    for (n, a), (_, b) in zip(donor.encoder.state_dict().items(), model.encoder.state_dict().items()):
        assert torch.equal(a, b), n

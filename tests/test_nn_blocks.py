import torch

from nmtgminor_b200 import nn as N


def test_rotary_preserves_norm_and_relative_phase():
    rot = N.RotaryEncoder(8, 32)
    x = torch.randn(1, 2, 10, 8)
    y = rot(x)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    q, k = torch.randn(1, 1, 1, 8), torch.randn(1, 1, 1, 8)
    a = (rot(q, 3) * rot(k, 5)).sum()
    b = (rot(q, 10) * rot(k, 12)).sum()
    assert torch.allclose(a, b, atol=1e-4)          # depends on the distance only


def test_masks():
    m = N.CausalAttentionMaskFactory()(3, 5, "cpu")
    assert m.shape == (3, 5) and m[0, 3] == float("-inf") and m[0, 2] == 0 and m[2, 4] == 0
    a = N.ALiBiMaskFactory(4)(4, 4, "cpu")
    assert a.shape == (4, 4, 4) and a[0, 3, 0] < a[0, 3, 2] <= 0 and a[0, 0, 1] == float("-inf")
    assert torch.allclose(N.ALiBiMaskFactory.slopes(8)[0], torch.tensor(0.5))


def test_rmsnorm_and_glu():
    x = torch.randn(2, 5, 16)
    y = N.RMSNorm(16)(x)
    assert torch.allclose(y.pow(2).mean(-1), torch.ones(2, 5), atol=1e-3)
    ffn = N.GLUFeedForwardNetwork(16, 64, inner_dim_to_multiple=32)
    assert ffn.inner_dim % 32 == 0 and ffn(x).shape == x.shape


def test_nllb_incremental_decoding_matches_full_forward():
    torch.manual_seed(0)
    cfg = N.NllbConfig(model_dim=32, max_seq_len=64, vocabulary_size=50, num_encoder_layers=2, num_decoder_layers=2,
                       num_encoder_attn_heads=4, num_decoder_attn_heads=4, ffn_inner_dim=64, dropout_p=0.0)
    model = N.create_nllb_model(cfg).eval()
    src = torch.randint(2, 50, (2, 7))
    src_len = torch.tensor([7, 5])
    tgt = torch.randint(2, 50, (2, 6))
    full = model(src, src_len, tgt)
    enc, mask = model.encode(src, src_len)
    state = {}
    steps = [model.decode(tgt[:, t:t + 1], enc, mask, state=state) for t in range(6)]
    assert torch.allclose(torch.cat(steps, 1), full, atol=1e-4)
    out = model.greedy(src, src_len, bos=2, eos=3, max_len=5)
    assert out.shape[0] == 2 and out.shape[1] <= 6


def test_llama_grouped_kv_and_generation():
    torch.manual_seed(0)
    cfg = N.LLaMAConfig(model_dim=32, max_seq_len=64, vocabulary_size=40, num_layers=2, num_attn_heads=4, num_key_value_heads=2,
                        ffn_inner_dim=64, ffn_inner_dim_to_multiple=16, dropout_p=0.0)
    model = N.create_llama_model(cfg).eval()
    toks = torch.randint(0, 40, (2, 9))
    full = model(toks)
    state = {}
    a = model(toks[:, :5], state=state)
    b = model(toks[:, 5:], state=state)
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-4)
    assert model.generate(toks[:, :3], 4).shape == (2, 7)
    sd = {"tok_embeddings.weight": 0, "layers.0.attention.wq.weight": 1, "layers.1.feed_forward.w3.weight": 2, "norm.weight": 3,
          "output.weight": 4, "rope.freqs": 5}
    conv = N.convert_llama_state_dict(sd)
    keys = set(model.state_dict().keys())
    assert set(conv.keys()) <= keys, set(conv.keys()) - keys


def test_unity_adaptor_shortens_sequences_and_masks():
    torch.manual_seed(0)
    adaptor = N.UnitYEncoderAdaptor(32, num_layers=1, num_heads=4, kernel_size=8, stride=8, dropout_p=0.0).eval()
    x = torch.randn(2, 64, 32)
    pad = torch.zeros(2, 64, dtype=torch.bool)
    pad[1, 40:] = True
    y, mask = adaptor(x, pad)
    assert y.shape == (2, 9, 32) and mask.shape == (2, 9)
    assert (~mask).sum(1).tolist() == [9, 6]

    class Inner(torch.nn.Module):
        def forward(self, feats, padding_mask=None):
            return feats, padding_mask
    enc = N.SeamlessSpeechEncoder(Inner(), adaptor)
    z, m2 = enc(x, pad)
    assert torch.allclose(z, y) and torch.equal(m2, mask)

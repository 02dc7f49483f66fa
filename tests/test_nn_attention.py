"""Pluggable attention of the typed building blocks: SDPA variants, weight hooks, default factory, LayerDrop list."""
import math

import torch

from nmtgminor_b200.nn.blocks import (AttentionWeightStoreHook, ModuleList, NaiveSDPA, RelativePositionalEncoding,
                                      RelativePositionSDPA, ShawRelativePositionSDPA, StandardMultiheadAttention, TorchSDPA,
                                      create_default_sdpa, default_sdpa_factory)


def _qkv(B=2, h=3, T=7, d=8, seed=0):
    torch.manual_seed(seed)
    return torch.randn(B, h, T, d), torch.randn(B, h, T, d), torch.randn(B, h, T, d)


def test_torch_and_naive_sdpa_agree_and_return_weights_on_request():
    q, k, v = _qkv()
    mask = torch.zeros(7, 7).masked_fill(torch.ones(7, 7).triu(1).bool(), float("-inf"))
    a, wa = TorchSDPA()(q, k, v, mask)
    b, wb = NaiveSDPA()(q, k, v, mask, needs_weights=True)
    assert wa is None and wb.shape == (2, 3, 7, 7)
    assert torch.allclose(a, b, atol=1e-5) and torch.allclose(wb.sum(-1), torch.ones(2, 3, 7), atol=1e-5)
    assert float(wb[0, 0, 0, 1:].abs().max()) == 0.0


def test_relative_position_sdpa_matches_the_explicit_sum():
    q, k, v = _qkv(T=5)
    sdpa = RelativePositionSDPA(24, 3, RelativePositionalEncoding(24, 4)).eval()     # the table grows from 4 to 5
    out, w = sdpa(q, k, v, needs_weights=True)
    T, d = 5, 8
    enc = sdpa.pos_encoding(T)                                                       # offsets T-1 .. -(T-1)
    r = sdpa.r_proj(enc).view(2 * T - 1, 3, d)
    scores = torch.zeros(2, 3, T, T)
    for i in range(T):
        for j in range(T):
            rel = r[(T - 1) - (i - j)]                                               # the encoding of offset i - j
            scores[:, :, i, j] = (((q[:, :, i] + sdpa.u_bias) * k[:, :, j]).sum(-1) + ((q[:, :, i] + sdpa.v_bias) * rel[None]).sum(-1))
    ref_w = torch.softmax(scores * d ** -0.5, -1)
    enc_offsets = torch.arange(T - 1, -T, -1)
    assert int(enc_offsets[(T - 1) - (4 - 2)]) == 4 - 2
    assert torch.allclose(w, ref_w, atol=1e-5) and torch.allclose(out, ref_w @ v, atol=1e-5)


def test_shaw_relative_position_sdpa():
    q, k, v = _qkv(T=6)
    sdpa = ShawRelativePositionSDPA(24, 3, max_left_rel_pos=2, max_right_rel_pos=1, use_rel_pos_values=True).eval()
    out, w = sdpa(q, k, v, needs_weights=True)
    idx = sdpa.rel_indices(6, 6, q.device)
    assert idx[0].tolist() == [2, 3, 3, 3, 3, 3] and idx[5].tolist() == [0, 0, 0, 0, 1, 2]
    scores = torch.einsum("bhqd,bhkd->bhqk", q, k) + torch.einsum("bhqd,qkd->bhqk", q, sdpa.rel_k_embed(idx))
    ref_w = torch.softmax(scores * 8 ** -0.5, -1)
    ref = ref_w @ v + torch.einsum("bhqk,qkd->bhqd", ref_w, sdpa.rel_v_embed(idx))
    assert torch.allclose(w, ref_w, atol=1e-5) and torch.allclose(out, ref, atol=1e-5)
    # incremental use: one query against six keys sees the offsets of the last position
    assert sdpa.rel_indices(1, 6, q.device).tolist() == [idx[5].tolist()]


def test_weight_hook_and_default_factory():
    torch.manual_seed(0)
    mha = StandardMultiheadAttention(32, 4).eval()
    assert isinstance(mha.sdpa, TorchSDPA)
    x = torch.randn(2, 5, 32)
    plain = mha(x)
    hook = AttentionWeightStoreHook()
    handle = mha.register_attn_weight_hook(hook)
    hooked = mha(x)
    assert torch.allclose(plain, hooked, atol=1e-5)
    assert len(hook.storage) == 1 and hook.storage[0][1].shape == (2, 4, 5, 5)
    handle.remove()
    mha(x)
    assert len(hook.storage) == 1
    with default_sdpa_factory(lambda attn_dropout_p=0.0: ShawRelativePositionSDPA(32, 4, 3, attn_dropout_p=attn_dropout_p)):
        shaw = StandardMultiheadAttention(32, 4)
        assert isinstance(shaw.sdpa, ShawRelativePositionSDPA) and isinstance(create_default_sdpa(), ShawRelativePositionSDPA)
    assert isinstance(create_default_sdpa(), TorchSDPA)
    assert shaw(x).shape == (2, 5, 32)


def test_module_list_layer_drop():
    layers = ModuleList([torch.nn.Linear(4, 4) for _ in range(200)], drop_p=0.25)
    layers.train()
    g = torch.Generator().manual_seed(0)
    kept = sum(1 for _ in layers.drop_iter(g))
    assert 120 < kept < 180
    layers.eval()
    assert sum(1 for _ in layers.drop_iter()) == 200
    assert layers.drop_p == 0.25

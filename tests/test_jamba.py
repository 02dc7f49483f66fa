"""Jamba blocks against plain statements of the same formulas."""
import math

import torch

from nmtgminor_b200.models.jamba import (JambaAttention, JambaAttentionDecoderLayer, JambaRMSNorm, JambaSparseMoeBlock, KVCache,
                                         load_balancing_loss)


def _plain_gqa(m, x, lengths):
    B, T, H = x.shape
    h, hk, d = m.num_heads, m.num_key_value_heads, m.head_dim
    q = m.q_proj(x).view(B, T, h, d).transpose(1, 2)
    k = m.k_proj(x).view(B, T, hk, d).transpose(1, 2).repeat_interleave(h // hk, 1)
    v = m.v_proj(x).view(B, T, hk, d).transpose(1, 2).repeat_interleave(h // hk, 1)
    s = q @ k.transpose(-1, -2) / math.sqrt(d)
    mask = torch.ones(T, T, dtype=torch.bool).tril()[None, None] & (torch.arange(T)[None, :] < lengths[:, None])[:, None, None, :]
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    out = m.o_proj((p @ v).transpose(1, 2).reshape(B, T, H))
    return out * (torch.arange(T)[None, :] < lengths[:, None])[..., None]


def test_grouped_query_attention_matches_plain_statement_and_cache_matches_full_pass():
    torch.manual_seed(0)
    m = JambaAttention(48, 6, 2).eval()
    x = torch.randn(3, 7, 48)
    lengths = torch.tensor([7, 4, 1])
    got = m(x, lengths)
    want = _plain_gqa(m, x, lengths)
    assert torch.allclose(got, want, atol=1e-5)
    # incremental decoding: a prefix of 4 tokens, then three single tokens
    full = m(x[:1])
    cache = KVCache()
    parts = [m(x[:1, :4], cache=cache)] + [m(x[:1, t:t + 1], cache=cache) for t in range(4, 7)]
    assert torch.allclose(torch.cat(parts, 1), full, atol=1e-5)
    assert cache.seen(0) == 7


def test_rms_norm():
    torch.manual_seed(1)
    n = JambaRMSNorm(16, eps=1e-5)
    with torch.no_grad():
        n.weight.uniform_(0.5, 1.5)
    x = torch.randn(5, 16)
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * n.weight
    assert torch.allclose(n(x), want, atol=1e-6)
    assert n(x.bfloat16()).dtype == torch.bfloat16


def test_moe_block_sums_the_chosen_experts():
    torch.manual_seed(2)
    moe = JambaSparseMoeBlock(12, 20, num_experts=4, top_k=2)
    x = torch.randn(2, 5, 12)
    out, logits = moe(x)
    assert logits.shape == (10, 4)
    flat = x.view(-1, 12)
    p = torch.softmax(logits, -1)
    want = torch.zeros_like(flat)
    for t in range(10):
        w, e = p[t].topk(2)
        for wi, ei in zip(w, e):
            want[t] += wi * moe.experts[int(ei)](flat[t])
    assert torch.allclose(out.view(-1, 12), want, atol=1e-5)


def test_load_balancing_loss_formula_and_mask():
    torch.manual_seed(3)
    E, k = 4, 2
    logits = tuple(torch.randn(6, E) for _ in range(3))
    got = load_balancing_loss(logits, E, k)
    cat = torch.cat(logits, 0)
    p = torch.softmax(cat, -1)
    chosen = p.topk(k, -1).indices
    want = 0.0
    for slot in range(k):
        for e in range(E):
            want += float((chosen[:, slot] == e).float().mean()) * float(p[:, e].mean())
    assert abs(float(got) - want * E) < 1e-5
    # a uniform router gives exactly top_k... no: f_e sums to 1 per slot and P_e = 1/E, so the loss is k
    uniform = (torch.zeros(8, E),)
    assert abs(float(load_balancing_loss(uniform, E, k)) - k) < 1e-5
    # padding rows do not count
    mask = torch.tensor([[1, 1, 0], [1, 0, 0]])
    masked = load_balancing_loss(logits, E, k, attention_mask=mask)
    keep = mask.reshape(-1).bool()
    kept = tuple(l[keep] for l in logits)
    assert abs(float(masked) - float(load_balancing_loss(kept, E, k))) < 1e-5
    assert load_balancing_loss(None, E) == 0


def test_decoder_layer_runs_and_backpropagates():
    torch.manual_seed(4)
    layer = JambaAttentionDecoderLayer(32, 4, 2, 64, num_experts=4, top_k=2)
    x = torch.randn(2, 6, 32, requires_grad=True)
    y, logits = layer(x, torch.tensor([6, 3]))
    (y.square().mean() + 0.01 * load_balancing_loss((logits,), 4, 2)).backward()
    assert x.grad is not None and all(p.grad is not None for p in layer.self_attn.parameters())
    dense = JambaAttentionDecoderLayer(32, 4, 4, 64)
    y2, none = dense(x.detach())
    assert none is None and y2.shape == x.shape

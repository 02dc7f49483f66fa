"""Plain PyTorch restatements of the fused ops: the CPU path and the numerical oracle of the tests.

Nothing here is tuned; every function states the mathematics of its CUDA counterpart in the most direct
way.  Packed variable-length attention is evaluated by padding to ``[B, T, heads, d]``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _act(x, act_id):
    if act_id == 0:
        return x
    if act_id == 1:
        return torch.relu(x)
    if act_id == 2:
        return F.gelu(x)
    if act_id == 3:
        return F.silu(x)
    raise ValueError("unknown activation id %r" % (act_id,))


def linear(x, weight, bias, act_id, dropout_p, residual):
    y = F.linear(x, weight.to(x.dtype), bias.to(x.dtype) if bias is not None else None)
    y = _act(y, act_id)
    if dropout_p > 0:
        y = F.dropout(y, dropout_p, True)
    if residual is not None:
        y = y + residual
    return y


def layer_norm(x, weight, bias, eps):
    return F.layer_norm(x, (x.shape[-1],), weight.to(x.dtype), bias.to(x.dtype), eps)


def dropout_add(x, residual, p):
    y = F.dropout(x, p, True) if p > 0 else x
    return y if residual is None else y + residual


def embedding(tokens, table, positions, pos_table, scale, p, pad_idx):
    out = F.embedding(tokens, table) * scale
    if pos_table is not None:
        pos = positions if positions is not None else torch.zeros_like(tokens)
        out = out + F.embedding(pos.clamp(0, pos_table.shape[0] - 1), pos_table).to(out.dtype)
    if p > 0:
        out = F.dropout(out, p, True)
    return out


def pad_packed(x, cu, max_len):
    """[N, ...] packed rows -> [B, max_len, ...] zero padded, plus a [B, max_len] validity mask."""
    cu_l = cu.tolist()
    B = len(cu_l) - 1
    out = x.new_zeros((B, max_len) + tuple(x.shape[1:]))
    mask = torch.zeros((B, max_len), dtype=torch.bool, device=x.device)
    for b in range(B):
        n = cu_l[b + 1] - cu_l[b]
        out[b, :n] = x[cu_l[b]:cu_l[b + 1]]
        mask[b, :n] = True
    return out, mask


def unpad_packed(xp, cu, total_rows):
    cu_l = cu.tolist()
    out = xp.new_zeros((total_rows,) + tuple(xp.shape[2:]))
    for b in range(len(cu_l) - 1):
        n = cu_l[b + 1] - cu_l[b]
        out[cu_l[b]:cu_l[b + 1]] = xp[b, :n]
    return out


def attention(q, k, v, cu_q, cu_k, heads, causal, dropout_p, scale=None, return_probs=False, bias=None):
    """softmax(scale * Q K^T + bias + masks) V per sequence and head; rows outside every sequence are zero.  ``bias``:
    optional ``[batch, heads, >= max_q, >= max_k]`` additive term."""
    d = q.shape[1] // heads
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    lq = (cu_q[1:] - cu_q[:-1]).tolist()
    lk = (cu_k[1:] - cu_k[:-1]).tolist()
    mq, mk = max(lq + [1]), max(lk + [1])
    qp, qm = pad_packed(q.view(q.shape[0], heads, d), cu_q, mq)
    kp, km = pad_packed(k.view(k.shape[0], heads, d), cu_k, mk)
    vp, _ = pad_packed(v.view(v.shape[0], heads, d), cu_k, mk)
    wt = torch.float64 if q.dtype == torch.float64 else torch.float32        # fp64 inputs (gradient checks) stay in fp64
    s = torch.einsum("bqhd,bkhd->bhqk", qp.to(wt), kp.to(wt)) * scale
    if bias is not None:
        s = s + bias[:, :, :mq, :mk].to(wt)
    s = s.masked_fill(~km[:, None, None, :], float("-inf"))
    if causal:
        tri = torch.ones(mq, mk, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~tri[None, None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0:
        p = F.dropout(p, dropout_p, True)
    o = torch.einsum("bhqk,bkhd->bqhd", p, vp.to(wt)).to(q.dtype)
    out = unpad_packed(o.reshape(o.shape[0], o.shape[1], heads * d), cu_q, q.shape[0])
    if return_probs:
        return out, p
    return out


def cross_entropy(logits, labels, smoothing, pad_idx):
    """Summed label-smoothed CE: (1-eps) * nll + eps * (lse - mean(logits)), pad rows excluded."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = labels != pad_idx
    safe = labels.clamp(0, logits.shape[1] - 1)
    nll = lse - lf.gather(1, safe[:, None]).squeeze(1)
    smooth = lse - lf.mean(dim=-1)
    row = ((1.0 - smoothing) * nll + smoothing * smooth) * valid
    correct = ((lf.argmax(dim=-1) == labels) & valid).sum().float().reshape(1)
    return row.sum().reshape(1), correct, row


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s):
        ctx.save_for_backward(s)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        (s,) = ctx.saved_tensors
        return g * s, None


def scale_gradient(x, s):
    """Identity in forward; multiplies the gradient by ``s`` in backward."""
    return _ScaleGrad.apply(x, s)


def adamw_step(master, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, max_grad_norm=0.0,
               decoupled=True):
    """One Adam(W) step on flat fp32 tensors (the oracle of the flat optimiser kernel)."""
    g = grad * grad_scale
    if max_grad_norm > 0:
        norm = g.norm()
        if norm > max_grad_norm:
            g = g * (max_grad_norm / (norm + 1e-6))
    if not decoupled and weight_decay:
        g = g + weight_decay * master
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mhat = m / (1 - beta1 ** step)
    denom = (v / (1 - beta2 ** step)).sqrt() + eps
    upd = mhat / denom
    if decoupled and weight_decay:
        upd = upd + weight_decay * master
    master.add_(upd, alpha=-lr)
    return master

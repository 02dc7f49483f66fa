"""Sequence-model ops: transducer joint and loss, diagonal complex linear recurrence (LRU), S4 Cauchy kernel
coefficients, softmax with key mask and dropout.

Each op runs the sm_100a kernel of ``csrc/sequence_kernels.cu`` on CUDA tensors and a plain PyTorch restatement
(``*_reference``) on CPU; the restatements are also the oracles of the GPU tests.

Reference behaviour: onmt/modules/transducer.py:1-230 (``TransducerJoint`` / ``TransducerLoss`` wrappers over
``transducer_joint_cuda`` / ``transducer_loss_cuda``), onmt/modules/extensions/blru/blru.py:19-120 (``BLRUFunction``,
``BLRU``), onmt/models/speech_recognizer/mssm/ssm_kernel/ssm_kernel_coefficient.py:31-110, and the softmax variants of
onmt/modules/extensions/multihead_attn/softmax_apex.h used by the attention modules when probabilities are returned.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn as nn

from . import _Rng, ext, next_stream


def _k(name):
    from . import LAUNCHES
    LAUNCHES[0] += 1
    return getattr(ext(), name)


# ------------------------------------------------------------------------------------------------------------
# transducer joint
def batch_offsets(f_len: torch.Tensor, g_len: torch.Tensor) -> torch.Tensor:
    """Inclusive prefix sums of ``f_len * g_len``: where every sentence ends in the packed [rows, H] lattice."""
    return torch.cumsum(f_len.long() * g_len.long(), 0)


def transducer_joint_reference(f, g, f_len, g_len, relu=False, dropout_mask=None, pack_output=False):
    h = f[:, :, None, :].float() + g[:, None, :, :].float()
    if relu:
        h = torch.relu(h)
    if dropout_mask is not None:
        h = h * dropout_mask
    B, T, U, _ = h.shape
    valid = (torch.arange(T, device=f.device)[None, :, None] < f_len[:, None, None]) & \
            (torch.arange(U, device=f.device)[None, None, :] < g_len[:, None, None])
    if pack_output:
        return torch.cat([h[b, :int(f_len[b]), :int(g_len[b])].reshape(-1, h.shape[-1]) for b in range(B)], 0).to(f.dtype)
    return (h * valid[..., None]).to(f.dtype)


class _JointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f, g, f_len, g_len, offsets, packed_rows, relu, p, seed, stream):
        out = _k("joint_fwd")(f.contiguous(), g.contiguous(), f_len, g_len, offsets, packed_rows, relu, p, seed, stream)
        ctx.save_for_backward(f_len, g_len, offsets if offsets is not None else f_len, out if relu else f_len)
        ctx.cfg = (f.shape[1], g.shape[1], relu, p, seed, stream, offsets is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        f_len, g_len, offsets, out = ctx.saved_tensors
        T, U, relu, p, seed, stream, packed = ctx.cfg
        df, dg = _k("joint_bwd")(dout.contiguous(), out if relu else None, f_len, g_len, offsets if packed else None, T, U, relu,
                                 p, seed, stream, 1.0)
        return df, dg, None, None, None, None, None, None, None, None


class TransducerJoint(nn.Module):
    """``h[b, t, u] = dropout(relu(f[b, t] + g[b, u]))``; ``pack_output`` drops the padding of every sentence and
    returns ``[sum_b f_len[b] * g_len[b], H]`` rows (sentence b ends at ``batch_offset[b]``)."""

    def __init__(self, pack_output: bool = False, relu: bool = False, dropout: bool = False, dropout_prob: float = 0.0):
        super().__init__()
        self.pack_output, self.relu = pack_output, relu
        self.dropout_prob = dropout_prob if dropout else 0.0

    def forward(self, f, g, f_len, g_len, batch_offset=None, packed_batch: int = 0):
        p = self.dropout_prob if self.training else 0.0
        f_len, g_len = f_len.int(), g_len.int()
        if not f.is_cuda:
            mask = None
            if p > 0:
                shape = (f.shape[0], f.shape[1], g.shape[1], f.shape[2])
                mask = (torch.rand(shape) >= p).float() / (1 - p)
            return transducer_joint_reference(f, g, f_len, g_len, self.relu, mask, self.pack_output)
        offsets = None
        if self.pack_output:
            offsets = batch_offset.long() if batch_offset is not None else batch_offsets(f_len, g_len)
            if not packed_batch:
                packed_batch = int(offsets[-1].item())
        return _JointFn.apply(f, g, f_len, g_len, offsets, packed_batch, self.relu, p, _Rng.seed, next_stream())


# ------------------------------------------------------------------------------------------------------------
# transducer loss
def transducer_loss_reference(x, label, f_len, y_len, blank_idx):
    """x: log-probabilities [B, T, U, V]; returns the negative log-likelihood of every sentence ([B])."""
    B = x.shape[0]
    losses = []
    for b in range(B):
        T, U = int(f_len[b]), int(y_len[b]) + 1
        neg_inf = torch.tensor(float("-inf"), dtype=x.dtype, device=x.device)
        alpha = [[None] * U for _ in range(T)]
        for t in range(T):
            for u in range(U):
                if t == 0 and u == 0:
                    alpha[t][u] = torch.zeros((), dtype=x.dtype, device=x.device)
                    continue
                a = alpha[t - 1][u] + x[b, t - 1, u, blank_idx] if t > 0 else neg_inf
                c = alpha[t][u - 1] + x[b, t, u - 1, label[b, u - 1]] if u > 0 else neg_inf
                alpha[t][u] = torch.logaddexp(a, c)
        losses.append(-(alpha[T - 1][U - 1] + x[b, T - 1, U - 1, blank_idx]))
    return torch.stack(losses)


class _RnntLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, label, f_len, y_len, offsets, max_f_len, blank, fuse_softmax):
        # with fuse_softmax the caller passes log-probabilities and receives the gradient of the logits
        alpha, beta, loss = _k("rnnt_loss_fwd")(x, label, f_len, y_len, offsets, max_f_len, blank)
        ctx.save_for_backward(x, alpha, beta, label, f_len, y_len, offsets if offsets is not None else f_len)
        ctx.cfg = (blank, fuse_softmax, offsets is not None)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x, alpha, beta, label, f_len, y_len, offsets = ctx.saved_tensors
        blank, fuse, packed = ctx.cfg
        dx = _k("rnnt_loss_bwd")(x, dloss.contiguous().float(), alpha, beta, label, f_len, y_len, offsets if packed else None,
                                 blank, fuse)
        return dx, None, None, None, None, None, None, None


class TransducerLoss(nn.Module):
    """RNN-T negative log-likelihood per sentence.

    ``x`` holds log-probabilities, dense ``[B, T, U, V]`` or packed ``[rows, V]`` (``packed_input``).  With
    ``fuse_softmax_backward`` the returned gradient is taken with respect to the logits that produced ``x`` by
    ``log_softmax`` (so the caller's ``log_softmax`` must be excluded from autograd: pass ``x.detach()`` results of it
    and route the gradient to the logits yourself, or use ``forward_logits``).
    """

    def __init__(self, fuse_softmax_backward: bool = False, packed_input: bool = False):
        super().__init__()
        self.fuse, self.packed = fuse_softmax_backward, packed_input

    def forward(self, x, label, f_len, y_len, blank_idx, batch_offset=None, max_f_len=None):
        f_len, y_len, label = f_len.int(), y_len.int(), label.int().contiguous()
        if not x.is_cuda:
            assert not self.packed, "the CPU restatement takes dense input"
            return transducer_loss_reference(x.float(), label.long(), f_len, y_len, blank_idx)
        offsets = None
        if self.packed:
            offsets = batch_offset.long() if batch_offset is not None else batch_offsets(f_len, y_len + 1)
            T = int(max_f_len) if max_f_len is not None else int(f_len.max().item())
        else:
            T = x.shape[1]
        return _RnntLossFn.apply(x.float().contiguous(), label, f_len, y_len, offsets, T, blank_idx, self.fuse)

    def forward_logits(self, logits, label, f_len, y_len, blank_idx, batch_offset=None, max_f_len=None):
        """Loss from raw logits with the log-softmax backward folded into the loss gradient kernel."""
        if not logits.is_cuda:
            return self.forward(torch.log_softmax(logits.float(), -1), label, f_len, y_len, blank_idx)
        return _LogitsLoss.apply(logits, self, label, f_len, y_len, blank_idx, batch_offset, max_f_len)


class _LogitsLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, mod, label, f_len, y_len, blank, batch_offset, max_f_len):
        x = torch.log_softmax(logits.float(), -1).contiguous()
        f_len, y_len, label = f_len.int(), y_len.int(), label.int().contiguous()
        offsets = None
        if mod.packed:
            offsets = batch_offset.long() if batch_offset is not None else batch_offsets(f_len, y_len + 1)
            T = int(max_f_len) if max_f_len is not None else int(f_len.max().item())
        else:
            T = x.shape[1]
        alpha, beta, loss = _k("rnnt_loss_fwd")(x, label, f_len, y_len, offsets, T, blank)
        ctx.save_for_backward(x, alpha, beta, label, f_len, y_len, offsets if offsets is not None else f_len)
        ctx.cfg = (blank, offsets is not None, logits.dtype)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x, alpha, beta, label, f_len, y_len, offsets = ctx.saved_tensors
        blank, packed, dtype = ctx.cfg
        dz = _k("rnnt_loss_bwd")(x, dloss.contiguous().float(), alpha, beta, label, f_len, y_len, offsets if packed else None,
                                 blank, True)
        return dz.to(dtype), None, None, None, None, None, None, None


# ------------------------------------------------------------------------------------------------------------
# diagonal complex linear recurrence
def lru_scan_reference(lam, x, lengths, direction):
    """h_t = lam * h_(t-1) + x_t along the last axis of x [B, N, L] (complex); see ``lru_scan``."""
    B, N, L = x.shape
    if direction == 2:
        half = N // 2
        return torch.cat([lru_scan_reference(lam[:half], x[:, :half], lengths, 0),
                          lru_scan_reference(lam[half:], x[:, half:], lengths, 1)], 1)
    outs = []
    for b in range(B):
        n = int(lengths[b])
        seq = x[b, :, :n]
        if direction == 1:
            seq = seq.flip(-1)
        hs, h = [], torch.zeros(N, dtype=x.dtype, device=x.device)
        for t in range(n):
            h = lam * h + seq[:, t]
            hs.append(h)
        out = torch.stack(hs, -1) if hs else x.new_zeros(N, 0)
        if direction == 1:
            out = out.flip(-1)
        outs.append(torch.cat([out, x.new_zeros(N, L - n)], -1))
    return torch.stack(outs)


class _LruFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lam, x, lengths, direction):
        h = _k("lru_scan_fwd")(lam.contiguous(), x.contiguous(), lengths, direction)
        ctx.save_for_backward(lam, h, lengths)
        ctx.direction = direction
        return h

    @staticmethod
    def backward(ctx, grad_h):
        lam, h, lengths = ctx.saved_tensors
        dx, dlam = _k("lru_scan_bwd")(lam.contiguous(), grad_h.contiguous(), h, lengths, ctx.direction)
        return dlam, dx, None, None


def lru_scan(lam, x, lengths, direction: int = 0):
    """``lam`` [N] complex64, ``x`` [B, N, L] complex64, ``lengths`` [B]; direction 0 forward, 1 backward (from
    ``lengths[b]-1``), 2 first half of the channels forward and second half backward."""
    if not x.is_cuda:
        return lru_scan_reference(lam, x, lengths, direction)
    return _LruFn.apply(lam.to(torch.complex64), x.to(torch.complex64), lengths.int(), direction)


class BLRU(nn.Module):
    """Bidirectional linear recurrent unit: ``u`` [B, L, H] -> ``y`` [B, L, H] through N complex diagonal states
    with eigenvalues initialised on a ring (``r_min`` .. ``r_max``, phase up to ``max_phase``)."""

    def __init__(self, H: int, N: int, direction: int = 2, r_min: float = 0.0, r_max: float = 1.0, max_phase: float = 2 * math.pi):
        super().__init__()
        u1, u2 = torch.rand(N), torch.rand(N)
        self.nu_log = nn.Parameter(torch.log(-0.5 * torch.log(u1 * (r_max ** 2 - r_min ** 2) + r_min ** 2)))
        self.theta_log = nn.Parameter(torch.log(max_phase * u2))
        lam = torch.exp(-torch.exp(self.nu_log.detach()) + 1j * torch.exp(self.theta_log.detach()))
        gamma = torch.sqrt(1 - lam.abs() ** 2)[:, None]
        self.B = nn.Parameter(torch.randn(H, N, 2) / math.sqrt(2 * H) * gamma)
        self.C = nn.Parameter(torch.randn(2, N, H) / math.sqrt(N))
        self.direction = direction

    def forward(self, u, lengths):
        lam = torch.exp(-torch.exp(self.nu_log) + 1j * torch.exp(self.theta_log)).to(torch.complex64)
        bu = torch.view_as_complex(torch.einsum("blh,hnz->bnlz", u.float(), self.B).contiguous())   # [B, N, L]
        x = lru_scan(lam, bu, lengths, self.direction).transpose(1, 2)                            # [B, L, N]
        return (x.real @ self.C[0] - x.imag @ self.C[1]).to(u.dtype)


# ------------------------------------------------------------------------------------------------------------
# S4 Cauchy kernel coefficients
def cauchy_reference(a, b, c):
    """out[i, q, l, h] = sum_n a[i, q, h, n] / (b[q, l, h] - c[q, n])"""
    r = 1.0 / (b[None, :, :, :, None] - c[None, :, None, None, :])          # [1, Q, L, H, N]
    return (a[:, :, None, :, :] * r).sum(-1)


class _CauchyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, c):
        a, b, c = a.contiguous(), b.contiguous(), c.contiguous()
        ctx.save_for_backward(a, b, c)
        return _k("cauchy_fwd")(a, b, c)

    @staticmethod
    def backward(ctx, dout):
        a, b, c = ctx.saved_tensors
        da, db, dc = _k("cauchy_bwd")(a, b, c, dout.contiguous())
        return da, db, dc


def cauchy_kernel_coefficient(a, b, c):
    if not a.is_cuda:
        return cauchy_reference(a, b, c)
    return _CauchyFn.apply(a.to(torch.complex64), b.to(torch.complex64), c.to(torch.complex64))


def compute_kernel_coefficient(z, d, t, b, c):
    """S4 kernel coefficients in the reference's argument convention: ``z`` [L, 2] (real view of complex nodes),
    ``d`` [Q, N] diagonal, ``t`` [Q, H] time steps, ``b`` [Q, I, H, N], ``c`` [Q, C, H, N]  ->  [Q, I, C, L, H]."""
    zz = torch.einsum("l,qh->qlh", torch.view_as_complex(z.float().contiguous()), (1.0 / t.float()).to(torch.complex64))
    bc = torch.einsum("qihn,qchn->icqhn", b.to(torch.complex64), c.to(torch.complex64))
    I, C, Q, H, N = bc.shape
    coeff = cauchy_kernel_coefficient(bc.reshape(I * C, Q, H, N), zz, d.to(torch.complex64))
    return coeff.view(I, C, Q, zz.shape[1], H).permute(2, 0, 1, 3, 4)


# ------------------------------------------------------------------------------------------------------------
# softmax with key mask and dropout
def softmax_dropout_reference(x, pad_mask=None, rows_per_mask=1, scale=1.0, drop_mask=None):
    cols = x.shape[-1]
    s = x.float().reshape(-1, cols) * scale
    if pad_mask is not None:
        m = pad_mask.reshape(-1, cols).bool().repeat_interleave(rows_per_mask, 0)
        s = s.masked_fill(m, float("-inf"))
    y = torch.nan_to_num(torch.softmax(s, -1), nan=0.0).reshape(x.shape)
    yd = y * drop_mask if drop_mask is not None else y
    return yd.to(x.dtype), y.to(x.dtype)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pad_mask, rows_per_mask, scale, p, seed, stream):
        yd, y = _k("softmax_dropout_fwd")(x.contiguous(), pad_mask, rows_per_mask, scale, p, seed, stream)
        if p <= 0:
            y = yd.clone()      # without dropout the kernel returns one tensor; the two outputs must be distinct objects
        ctx.save_for_backward(y)
        ctx.cfg = (scale, p, seed, stream)
        ctx.mark_non_differentiable(y)
        return yd, y

    @staticmethod
    def backward(ctx, dyd, _dy):
        (y,) = ctx.saved_tensors
        scale, p, seed, stream = ctx.cfg
        return _k("softmax_dropout_bwd")(dyd.contiguous(), y, scale, p, seed, stream), None, None, None, None, None, None


class _SoftmaxRecomputeFn(torch.autograd.Function):
    """Same result as ``_SoftmaxFn`` but nothing of size ``x`` is kept for backward except ``x`` itself: the softmax is
    recomputed from the input there (the reference's "recompute" backward variants, softmax_apex.h: dispatch_*_backward_recompute)."""

    @staticmethod
    def forward(ctx, x, pad_mask, rows_per_mask, scale, p, seed, stream):
        yd, y = _k("softmax_dropout_fwd")(x.contiguous(), pad_mask, rows_per_mask, scale, p, seed, stream)
        ctx.save_for_backward(x, pad_mask) if pad_mask is not None else ctx.save_for_backward(x)
        ctx.cfg = (rows_per_mask, scale, p, seed, stream, pad_mask is not None)
        return yd

    @staticmethod
    def backward(ctx, dyd):
        rows_per_mask, scale, p, seed, stream, has_mask = ctx.cfg
        x = ctx.saved_tensors[0]
        pad_mask = ctx.saved_tensors[1] if has_mask else None
        yd, y = _k("softmax_dropout_fwd")(x.contiguous(), pad_mask, rows_per_mask, scale, p, seed, stream)
        y = y if p > 0 else yd
        return _k("softmax_dropout_bwd")(dyd.contiguous(), y, scale, p, seed, stream), None, None, None, None, None, None


def time_mask_from_lengths(lengths: torch.Tensor, cols: int) -> torch.Tensor:
    """Key mask (nonzero = masked) ``[len(lengths), cols]`` for rows that may look at their first ``lengths[i]`` columns."""
    return (torch.arange(cols, device=lengths.device)[None, :] >= lengths.to(torch.int64)[:, None]).to(torch.uint8)


def masked_softmax_dropout(x, *, pad_mask: Optional[torch.Tensor] = None, additive_mask: Optional[torch.Tensor] = None,
                           lengths: Optional[torch.Tensor] = None, rows_per_mask: int = 1, scale: float = 1.0, p: float = 0.0,
                           drop_mask: Optional[torch.Tensor] = None, recompute: bool = False, training: bool = True):
    """The softmax family of the reference's attention extensions (softmax_apex.h: plain, + dropout, + presampled dropout,
    additive-masked, time-masked, backward from the saved output or recomputed from the input) behind one call:

    * ``pad_mask`` (nonzero = masked, one row per ``rows_per_mask`` rows of ``x``) or ``lengths`` (time mask: row group i
      sees its first ``lengths[i]`` columns) or ``additive_mask`` (float, broadcastable to ``x``, added to the scaled scores);
    * ``p``: dropout drawn by the kernel from its counters, or ``drop_mask`` (presampled, already scaled by 1 / (1 - p));
    * ``recompute``: keep only ``x`` for backward and recompute the probabilities there.

    Returns the (dropped) probabilities.  On a GPU everything but the additive mask and the presampled dropout mask (one
    element-wise PyTorch op each) runs in the warp-per-row kernels."""
    cols = x.shape[-1]
    if lengths is not None:
        if pad_mask is not None:
            raise ValueError("give either pad_mask or lengths")
        pad_mask = time_mask_from_lengths(lengths, cols)
    if additive_mask is not None:
        x = x + (additive_mask / scale if scale != 1.0 else additive_mask).to(x.dtype)
    p_kernel = 0.0 if drop_mask is not None else (p if training else 0.0)
    if not x.is_cuda:
        drop = drop_mask
        if drop is None and p_kernel > 0:
            drop = (torch.rand(x.shape) >= p_kernel).float() / (1 - p_kernel)
        return softmax_dropout_reference(x, pad_mask, rows_per_mask, scale, drop)[0]
    if pad_mask is not None:
        pad_mask = pad_mask.to(torch.uint8).contiguous()
    if recompute:
        out = _SoftmaxRecomputeFn.apply(x, pad_mask, rows_per_mask, scale, p_kernel, _Rng.seed, next_stream())
    else:
        out = _SoftmaxFn.apply(x, pad_mask, rows_per_mask, scale, p_kernel, _Rng.seed, next_stream())[0]
    return out * drop_mask.to(out.dtype) if drop_mask is not None else out


def softmax_dropout(x, pad_mask: Optional[torch.Tensor] = None, rows_per_mask: int = 1, scale: float = 1.0, p: float = 0.0,
                    training: bool = True):
    """Returns ``(dropout(softmax(scale * x + mask)), softmax(...))`` over the last axis; ``pad_mask`` (nonzero = masked)
    has one row per ``rows_per_mask`` consecutive rows of ``x`` (e.g. heads * queries rows per sentence)."""
    p = p if training else 0.0
    if not x.is_cuda:
        drop = (torch.rand(x.shape) >= p).float() / (1 - p) if p > 0 else None
        return softmax_dropout_reference(x, pad_mask, rows_per_mask, scale, drop)
    if pad_mask is not None:
        pad_mask = pad_mask.to(torch.uint8).contiguous()
    return _SoftmaxFn.apply(x, pad_mask, rows_per_mask, scale, p, _Rng.seed, next_stream())

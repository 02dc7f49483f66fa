"""1-D convolution over channels-last sequences as a tensor-core GEMM without an im2col buffer.

For ``x`` [B, T, Ci] (channels last, time padded to a multiple of the stride) the im2col row of output frame
``(b, t)`` is the contiguous run ``x[b, t*s : t*s + k, :]``: ``k * Ci`` elements starting ``s * Ci`` elements after
the previous row.  That is an ordinary 2-D tensor whose rows overlap, which a TMA descriptor (row stride ``s * Ci``,
row length ``k * Ci``) reads directly, so the convolution is ONE ``gemm(A_view, W[Co, k*Ci])`` with the bias and the
activation in the epilogue.  If the driver refuses descriptors with overlapping rows the same result is produced
from ``k`` GEMMs over non-overlapping single-tap views.  The weight gradient is the transposed product over the same
view; the input gradient is ``k`` GEMMs that scatter each tap back into its strided slot.

Used for the wav2vec2 feature extractor layers after the first (512 channels, k 3 / 2, stride 2) and the Whisper
stem (80 -> 1280 k3, 1280 -> 1280 k3 s2), replacing cuDNN calls of the reference (onmt/models/speech_recognizer/
fairseq_wav2vec2/wav2vec2.py ``ConvFeatureExtractionModel``; onmt/models/whisper/whisper_encoder.py conv1 / conv2).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ACT_IDS, _act_backward, empty_rows, ext, fused_param, gemm

_OVERLAP_OK = [None]      # None = untested, True / False once the driver answered


def conv1d_reference(x, weight, bias=None, stride: int = 1, act: str = "none"):
    """x [B, T, Ci], weight [Co, Ci, k] -> [B, T_out, Co] (plain PyTorch)."""
    y = F.conv1d(x.transpose(1, 2).float(), weight.float(), None if bias is None else bias.float(), stride=stride).transpose(1, 2)
    if act == "gelu":
        y = F.gelu(y)
    elif act == "relu":
        y = F.relu(y)
    elif act in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype)


def _padded_input(x, k: int, s: int):
    """Copy x into a zero-tailed buffer whose time axis is a multiple of the stride; returns (flat [rows, Ci], Tp)."""
    B, T, Ci = x.shape
    Tp = (T + s - 1) // s * s
    buf = torch.zeros((B * Tp + k, Ci), dtype=torch.bfloat16, device=x.device)
    buf[:B * Tp].view(B, Tp, Ci)[:, :T].copy_(x)
    return buf, Tp


def _overlap_view(buf, M: int, k: int, s: int, Ci: int):
    return buf.as_strided((M, k * Ci), (s * Ci, 1))


def _tap_view(buf, M: int, tap: int, s: int, Ci: int):
    return buf.as_strided((M, Ci), (s * Ci, 1), storage_offset=tap * Ci)


class _Conv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_work, b_work, gw, gb, stride, act, need_dx):
        B, T, Ci = x.shape
        Co, _, k = w_work.shape
        s = stride
        buf, Tp = _padded_input(x, k, s)
        M = B * Tp // s
        wg = w_work.permute(0, 2, 1).reshape(Co, k * Ci).contiguous()          # [Co, k*Ci], tap-major like the rows of A
        out = empty_rows(M, Co, x.device)
        pre = empty_rows(M, Co, x.device) if act != 0 else None
        done = False
        if _OVERLAP_OK[0] is not False:
            try:
                gemm(_overlap_view(buf, M, k, s, Ci), wg, out, bias=b_work, preact=pre, act=act)
                _OVERLAP_OK[0] = done = True
            except RuntimeError as exc:
                if "cuTensorMapEncodeTiled" not in str(exc):
                    raise
                _OVERLAP_OK[0] = False
        if not done:
            acc = out if act == 0 else pre
            for tap in range(k):
                gemm(_tap_view(buf, M, tap, s, Ci), wg[:, tap * Ci:(tap + 1) * Ci], acc, bias=b_work if tap == 0 else None,
                     residual=acc if tap > 0 else None)
            if act != 0:
                a = pre.float()
                out.copy_((F.relu(a) if act == 1 else F.gelu(a) if act == 2 else F.silu(a)).to(out.dtype))
        T_out = (T - k) // s + 1
        ctx.save_for_backward(buf, wg, pre if pre is not None else out)
        ctx.cfg = (B, T, Tp, Ci, Co, k, s, act, T_out, need_dx, M)
        ctx.gw, ctx.gb = gw, gb
        return out.view(B, Tp // s, Co)[:, :T_out]

    @staticmethod
    def backward(ctx, dy):
        buf, wg, pre = ctx.saved_tensors
        B, T, Tp, Ci, Co, k, s, act, T_out, need_dx, M = ctx.cfg
        # frames past T_out (they straddle two utterances or the zero tail) received no gradient
        dz = torch.zeros((M, Co), dtype=torch.bfloat16, device=dy.device)
        dz.view(B, Tp // s, Co)[:, :T_out].copy_(dy)
        if act != 0:
            dz = _act_backward(dz, pre, act)
            dz.view(B, Tp // s, Co)[:, T_out:].zero_()
        if ctx.gw is not None:
            dwg = torch.zeros((Co, k * Ci), dtype=torch.float32, device=dy.device)
            if _OVERLAP_OK[0]:
                gemm(dz, _overlap_view(buf, M, k, s, Ci), dwg, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
            else:
                for tap in range(k):
                    gemm(dz, _tap_view(buf, M, tap, s, Ci), dwg[:, tap * Ci:(tap + 1) * Ci], a_mn_major=True, b_mn_major=True,
                         accumulate=True, allow_split_k=True)
            ctx.gw.add_(dwg.view(Co, k, Ci).permute(0, 2, 1))
        if ctx.gb is not None:
            ext().colsum(dz, ctx.gb)
        dx = None
        if need_dx:
            dbuf = torch.zeros_like(buf)
            for tap in range(k):
                # tap `tap` of every frame lands in its own strided slot; later taps add to what earlier taps wrote
                slot = _tap_view(dbuf, M, tap, s, Ci)
                gemm(dz, wg[:, tap * Ci:(tap + 1) * Ci], slot, b_mn_major=True, residual=slot if tap >= s else None)
            dx = dbuf[:B * Tp].view(B, Tp, Ci)[:, :T]
        return dx, None, None, None, None, None, None, None


def conv1d(x, weight, bias=None, stride: int = 1, act: str = "none", padding: int = 0):
    """Channels-last 1-D convolution: ``x`` [B, T, Ci], ``weight`` [Co, Ci, k] (the ``nn.Conv1d`` layout).

    Takes the GEMM path for parameters with bf16 working copies when ``stride * Ci`` and ``Ci`` are multiples of 8;
    anything else (the single-channel first wav2vec2 layer, grouped convolutions) runs ``F.conv1d``."""
    act_id = ACT_IDS[act]
    if padding:
        x = F.pad(x, (0, 0, padding, padding))
    Ci = x.shape[-1]
    if not (fused_param(weight) and x.is_cuda and Ci % 8 == 0 and (stride * Ci) % 8 == 0 and weight.shape[1] == Ci):
        return conv1d_reference(x, weight, bias, stride, act)
    gw = weight.main_grad if weight.requires_grad else None
    gb = bias.main_grad if (bias is not None and bias.requires_grad) else None
    xin = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if not torch.is_grad_enabled():
        gw = gb = None
    return _Conv1dFn.apply(xin, weight.work, bias.work if bias is not None else None, gw, gb, int(stride), act_id,
                           bool(x.requires_grad and torch.is_grad_enabled()))

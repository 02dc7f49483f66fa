"""Functional op layer.

Every hot op of the framework has two implementations with the same signature:

* the sm_100a kernels of ``csrc/`` (tcgen05 GEMM with fused epilogues, tcgen05 variable-length attention,
  LayerNorm, fused label-smoothed cross-entropy, embedding, dropout-add, flat AdamW), wrapped in
  ``torch.autograd.Function`` objects whose backward passes are hand-derived and which write weight
  gradients straight into the flat fp32 gradient buffer (``param.main_grad``) instead of returning them;
* a plain PyTorch restatement (``reference.py``) used on CPU, as the numerical oracle in the tests, and
  nowhere on a GPU hot path.

A parameter takes the fused path when it carries a bf16 working copy (``param.work``, attached by
``nmtgminor_b200.parallel.flat.FlatParameterStore``) that lives on a CUDA device.  On a CUDA device the
extension must be present: a missing or unloadable shared object raises instead of silently falling back.

The op set mirrors what the reference implements as separate extensions: self / encoder-decoder
attention (onmt/modules/optimized/self_attention_func.py:53-504, encdec_attention_func_bias.py), fused MLP
(onmt/modules/mlp/mlp.py:55-211), LayerNorm (onmt/modules/layer_norm.py:29-168), fused cross-entropy
(onmt/modules/optimized/softmax_xentropy.py:5-28), dropout-add (onmt/modules/optimized/dropout_add.py:32-90)
and the fused optimiser (onmt/modules/optimized/fused_adam.py:4-191).
"""
from __future__ import annotations

import importlib.util
import math
import os
import threading
from typing import Optional

import torch
import torch.nn.functional as F

from . import reference as ref

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_nmtg_b200_C.so")
_ext = None
_ext_err: Optional[str] = None
_lock = threading.Lock()

ACT_IDS = {"none": 0, None: 0, "relu": 1, "gelu": 2, "silu": 3, "swish": 3}
_ACT_BWD = {1: 5, 2: 6, 3: 7}


def load_extension(build_if_missing: bool = True):
    """Import the in-tree shared object (building it first when it is absent and nvcc exists)."""
    global _ext, _ext_err
    with _lock:
        if _ext is not None:
            return _ext
        try:
            if not os.path.exists(_SO) and build_if_missing:
                from .build import build
                build()
            spec = importlib.util.spec_from_file_location("_nmtg_b200_C", _SO)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _ext = mod
        except Exception as exc:  # noqa: BLE001 - reported to the caller below
            _ext_err = repr(exc)
            _ext = None
        return _ext


def extension_available() -> bool:
    return load_extension(build_if_missing=False) is not None


_KERNEL_CALLS = {"gemm": 1, "layernorm_fwd": 1, "layernorm_bwd": 1, "xent_fused": 1, "dropout_add": 1,
                 "dropout_colsum": 1, "embed_fwd": 1, "embed_bwd": 1, "colsum": 1, "sq_norm": 1, "adamw_flat": 1, "cast_f32_bf16": 1, "attn_fwd": 1,
                 "attn_bwd": 1, "update_pieces": 1, "act_backward": 1}
LAUNCHES = [0]   # kernels of this extension enqueued so far (Python-side count of launcher calls)


class _CountingExt:
    """Forwards to the extension module and counts calls that enqueue one of its kernels."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        f = self._cache.get(name)
        if f is None:
            raw = getattr(self._mod, name)
            n = _KERNEL_CALLS.get(name, 0)
            if n:
                def f(*a, _raw=raw, _n=n, **k):
                    LAUNCHES[0] += _n
                    return _raw(*a, **k)
            else:
                f = raw
            self._cache[name] = f
        return f


_proxy = None


def ext():
    global _proxy
    if _proxy is not None:
        return _proxy
    e = load_extension()
    if e is None:
        raise RuntimeError("the sm_100a extension %s could not be loaded (%s); build it with "
                           "`python -m nmtgminor_b200.ops.build`" % (_SO, _ext_err))
    _proxy = _CountingExt(e)
    return _proxy


def fused_param(p) -> bool:
    w = getattr(p, "work", None)
    return w is not None and w.is_cuda


def check_status(device=None) -> int:
    """Read (and clear) the device status word; non-zero means a bounded wait inside a kernel gave up."""
    if not torch.cuda.is_available():
        return 0
    dev = torch.cuda.current_device() if device is None else device
    s = int(ext().read_status(dev))
    if s:
        ext().clear_status(dev)
    return s


# ---------------------------------------------------------------------------------------------------
# dropout bookkeeping: (seed, stream id per op call); masks are regenerated in backward from the same pair
# ---------------------------------------------------------------------------------------------------
class _Rng:
    seed = 1234
    counter = 0


def manual_seed(seed: int) -> None:
    _Rng.seed = int(seed) & 0x7FFFFFFFFFFFFFFF
    _Rng.counter = 0


def next_stream() -> int:
    _Rng.counter += 1
    return _Rng.counter


def reset_stream_counter() -> None:
    """Call at the start of each step so that op call i always gets stream id i (graph-replay safe)."""
    _Rng.counter = 0


def advance_device_seed(device=None, by: int = 1) -> None:
    """Adds `by` to the device-resident seed word (a tiny kernel, capturable in a CUDA graph)."""
    dev = torch.cuda.current_device() if device is None else device
    ext().get_seed_tensor(dev).add_(by)


# ---------------------------------------------------------------------------------------------------
# GEMM primitives
# ---------------------------------------------------------------------------------------------------
def gemm(a, b, out, *, a_mn_major=False, b_mn_major=False, bias=None, residual=None, aux=None, preact=None, act=0,
         dropout_p=0.0, seed=0, stream_id=0, alpha=1.0, accumulate=False, allow_split_k=False, split_k=0, force_bn=0,
         mask=None, colsum=None, gather=None):
    """out[M,N] = epilogue(alpha * A B^T) on the tcgen05 kernel (see csrc/ops_api.h: GemmDesc).  ``mask`` (int32
    [M, ceil(N/32)]) receives the sign bits of the output, or supplies them when ``act`` is the mask-backward id 8.
    ``colsum`` (fp32 [N]): the column sums of the bf16 output are added to it by the epilogue (bias gradients).
    ``gather``: record of a fully sharded weight (``parallel.fsdp.GatherInfo``) whose pieces this call pulls from
    their owners into ``b`` before (and while) it multiplies."""
    g = gather.pending() if gather is not None else None
    ext().gemm(a, a_mn_major, b, b_mn_major, out, bias, residual, aux, preact, int(act), float(dropout_p), int(seed),
               int(stream_id), float(alpha), bool(accumulate), bool(allow_split_k), int(split_k), int(force_bn), mask, colsum, g)
    return out


def _gather_of(weight):
    """The gather record of a fully sharded weight matrix, or None (replicated parameters)."""
    return getattr(weight, "_fsdp", None)


def empty_rows(rows: int, cols: int, device, dtype=torch.bfloat16):
    """[rows, cols] tensor whose row stride is rounded up to 16 bytes (kernels need aligned rows; e.g. vocabulary
    sizes that are not multiples of 8).  The result is a column slice of a wider buffer when padding is needed."""
    mult = 16 // torch.empty((), dtype=dtype).element_size()
    padded = (cols + mult - 1) // mult * mult
    t = torch.empty((rows, padded), dtype=dtype, device=device)
    return t if padded == cols else t[:, :cols]


def _track(x):
    """Input of a fused autograd node whose only gradients go to parameters (written straight into ``main_grad``):
    autograd records a node only if some tensor input requires grad, so an input that does not (frozen embeddings in
    front of trainable adapters, say) is replaced by a detached leaf that does."""
    return x if x.requires_grad else x.detach().requires_grad_(True)


def _keep_scale(p: float) -> float:
    """Dropout is byte-granular on the device: keep probability (256 - round(256 p)) / 256."""
    if p <= 0.0:
        return 1.0
    return 256.0 / (256 - int(p * 256.0 + 0.5))


class _LinearFn(torch.autograd.Function):
    """y = [residual +] dropout(act(x W^T + b)); weight/bias gradients go to the main_grad buffers."""

    @staticmethod
    def forward(ctx, x, w, bias, residual, gw, gb, act, dropout_p, seed, stream_id, need_input_grad, gather=None):
        M, N = x.shape[0], w.shape[0]
        y = empty_rows(M, N, x.device)
        z = empty_rows(M, N, x.device) if act != 0 else None  # pre-activation, needed by act'
        gemm(x, w, y, bias=bias, residual=residual, preact=z, act=act, dropout_p=dropout_p, seed=seed,
             stream_id=stream_id, gather=gather)
        ctx.save_for_backward(x, w, z)
        ctx.cfg = (act, dropout_p, seed, stream_id, residual is not None, bias is not None, need_input_grad)
        ctx.gw, ctx.gb = gw, gb
        ctx.gather = gather
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, z = ctx.saved_tensors
        act, p, seed, sid, has_res, has_bias, need_dx = ctx.cfg
        if dy.shape[1] % 8:
            padded = empty_rows(dy.shape[0], dy.shape[1], dy.device)
            padded.copy_(dy)
            dy = padded
        else:
            dy = dy.contiguous()
        want_gb = has_bias and ctx.gb is not None
        fused_gb = want_gb and act == 0 and p > 0.0 and _colsum_fusable(dy)
        if fused_gb:
            dz = ext().dropout_colsum(dy, p, seed, sid, ctx.gb)  # regenerated mask and bias gradient in one pass
        elif act != 0 and dy.numel() % 8 == 0:
            dz = ext().act_backward(dy, z, act, p, seed, sid)    # regenerated mask times act'(z) in one pass
        else:
            dz = ext().dropout_add(dy, None, p, seed, sid) if p > 0.0 else dy  # regenerates the forward mask
            if act != 0:
                dz = _act_backward(dz, z, act)
        if ctx.gw is not None:
            gemm(dz, x, ctx.gw, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
        if want_gb and not fused_gb:
            ext().colsum(dz, ctx.gb)
        dx = None
        if need_dx:
            dx = torch.empty((dy.shape[0], x.shape[1]), dtype=torch.bfloat16, device=dy.device)
            gemm(dz, w, dx, b_mn_major=True, gather=ctx.gather)
        return dx, None, None, (dy if has_res else None), None, None, None, None, None, None, None, None


def _colsum_fusable(dy):
    """The one-pass masked-gradient + bias-gradient kernel takes 16 * (8, 16, ..., 256) columns."""
    n = dy.shape[1]
    return dy.dim() == 2 and n % 128 == 0 and n <= 4096 and (n & (n - 1)) == 0


def _act_backward(dh, z, act):
    """dz = dh * act'(z) in PyTorch ops: the oracle of the ``act_backward`` kernel, and the path for element counts that are
    not a multiple of 8 (the FFN path fuses this step into a GEMM epilogue)."""
    a = z.float()
    if act == 1:
        g = (a > 0).float()
    elif act == 2:
        g = 0.5 * (1.0 + torch.erf(a * 0.7071067811865476)) + a * torch.exp(-0.5 * a * a) * 0.3989422804014327
    else:
        sg = torch.sigmoid(a)
        g = sg * (1.0 + a * (1.0 - sg))
    return (dh.float() * g).to(torch.bfloat16)


def linear(x, weight, bias=None, act="none", dropout_p=0.0, residual=None, training=True):
    """Fused Linear: ``[residual +] dropout(act(x @ weight.T + bias))`` on 2-D ``x``."""
    act_id = ACT_IDS[act] if not isinstance(act, int) else act
    p = float(dropout_p) if training else 0.0
    if fused_param(weight) and x.is_cuda:
        b = bias.work if bias is not None else None
        gw = getattr(weight, "main_grad", None) if weight.requires_grad else None
        gb = getattr(bias, "main_grad", None) if (bias is not None and bias.requires_grad) else None
        sid = next_stream() if p > 0 else 0
        need_dx = x.requires_grad
        xin = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        if not torch.is_grad_enabled() or not (need_dx or gw is not None):
            y = empty_rows(x.shape[0], weight.shape[0], x.device)
            return gemm(xin, weight.work, y, bias=b, residual=residual, act=act_id, dropout_p=p, seed=_Rng.seed,
                        stream_id=sid, gather=_gather_of(weight))
        return _LinearFn.apply(_track(xin), weight.work, b, residual, gw, gb, act_id, p, _Rng.seed, sid, need_dx,
                               _gather_of(weight))
    return ref.linear(x, weight, bias, act_id, p, residual)


class _MlpFn(torch.autograd.Function):
    """y = residual + D2( D1(act(x W1^T + b1)) W2^T + b2 ), five GEMM launches forward + backward.

    Every element-wise step rides in a GEMM epilogue: bias + activation + dropout (fc1), bias + dropout +
    residual (fc2), and in backward the activation gradient (and, for GELU/SiLU, the regenerated fc1
    dropout mask) is the epilogue of the fc2 data-gradient product.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, g, act, p1, p2, seed, sid1, sid2, gather1=None, gather2=None):
        M = x.shape[0]
        h = torch.empty((M, w1.shape[0]), dtype=torch.bfloat16, device=x.device)
        z = torch.empty_like(h) if act != 1 else None
        # ReLU: the epilogue also writes one sign bit per element (ReLU and dropout mask in one), which is all the
        # backward pass needs from h: 1/16 of the bytes of re-reading h
        bits = torch.empty((M, (w1.shape[0] + 31) // 32), dtype=torch.int32, device=x.device) if act == 1 else None
        gemm(x, w1, h, bias=b1, preact=z, act=act, dropout_p=p1, seed=seed, stream_id=sid1, mask=bits, gather=gather1)
        y = torch.empty((M, w2.shape[0]), dtype=torch.bfloat16, device=x.device)
        gemm(h, w2, y, bias=b2, residual=residual, dropout_p=p2, seed=seed, stream_id=sid2, gather=gather2)
        ctx.save_for_backward(x, w1, w2, h, z if z is not None else bits)
        ctx.cfg = (act, p1, p2, seed, sid1, sid2, residual is not None)
        ctx.g = g
        ctx.gathers = (gather1, gather2)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, h, z = ctx.saved_tensors
        act, p1, p2, seed, sid1, sid2, has_res = ctx.cfg
        gw1, gb1, gw2, gb2 = ctx.g
        dy = dy.contiguous()
        fused_gb2 = gb2 is not None and p2 > 0.0 and _colsum_fusable(dy)
        if fused_gb2:
            dz2 = ext().dropout_colsum(dy, p2, seed, sid2, gb2)
        else:
            dz2 = ext().dropout_add(dy, None, p2, seed, sid2) if p2 > 0.0 else dy
        if gw2 is not None:
            gemm(dz2, h, gw2, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
        if gb2 is not None and not fused_gb2:
            ext().colsum(dz2, gb2)
        dz1 = torch.empty_like(h)
        fused_gb1 = False
        if act == 1:   # the sign bits encode ReLU and the dropout mask; only the keep scale is missing
            # with more than 128 rows the CTA-pair kernel runs, whose epilogue can also sum the columns (fc1 bias gradient)
            fused_gb1 = gb1 is not None and dz2.shape[0] > 128 and dz1.shape[1] % 8 == 0
            gemm(dz2, w2, dz1, b_mn_major=True, act=8, mask=z, alpha=_keep_scale(p1), colsum=gb1 if fused_gb1 else None,
                 gather=ctx.gathers[1])
        else:
            gemm(dz2, w2, dz1, b_mn_major=True, aux=z, act=_ACT_BWD[act], dropout_p=p1, seed=seed, stream_id=sid1,
                 gather=ctx.gathers[1])
        if gw1 is not None:
            gemm(dz1, x, gw1, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
        if gb1 is not None and not fused_gb1:
            ext().colsum(dz1, gb1)
        dx = torch.empty_like(x)
        gemm(dz1, w1, dx, b_mn_major=True, gather=ctx.gathers[0])
        return (dx, None, None, None, None, (dy if has_res else None)) + (None,) * 9


def mlp(x, w1, b1, w2, b2, act="relu", dropout_p=0.0, out_dropout_p=0.0, residual=None, training=True):
    """Position-wise feed-forward block: ``[residual +] D(D(act(x W1^T + b1)) W2^T + b2)``."""
    act_id = ACT_IDS[act] if not isinstance(act, int) else act
    p1 = float(dropout_p) if training else 0.0
    p2 = float(out_dropout_p) if training else 0.0
    if fused_param(w1) and x.is_cuda and act_id in (1, 2, 3):
        xin = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        sid1 = next_stream() if p1 > 0 else 0
        sid2 = next_stream() if p2 > 0 else 0
        if torch.is_grad_enabled():
            g = tuple(getattr(t, "main_grad", None) if (t is not None and t.requires_grad) else None
                      for t in (w1, b1, w2, b2))
            return _MlpFn.apply(_track(xin), w1.work, b1.work if b1 is not None else None, w2.work,
                                b2.work if b2 is not None else None, residual, g, act_id, p1, p2, _Rng.seed, sid1, sid2,
                                _gather_of(w1), _gather_of(w2))
        h = torch.empty((x.shape[0], w1.shape[0]), dtype=torch.bfloat16, device=x.device)
        gemm(xin, w1.work, h, bias=b1.work if b1 is not None else None, act=act_id, gather=_gather_of(w1))
        y = torch.empty((x.shape[0], w2.shape[0]), dtype=torch.bfloat16, device=x.device)
        return gemm(h, w2.work, y, bias=b2.work if b2 is not None else None, residual=residual, gather=_gather_of(w2))
    h = ref.linear(x, w1, b1, act_id, p1, None)
    return ref.linear(h, w2, b2, 0, p2, residual)


# ---------------------------------------------------------------------------------------------------
# LayerNorm
# ---------------------------------------------------------------------------------------------------
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, b, gg, gb, eps):
        y, mean, rstd = ext().layernorm_fwd(x, g, b, eps)
        ctx.save_for_backward(x, mean, rstd, g)
        ctx.gg, ctx.gb = gg, gb
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd, g = ctx.saved_tensors
        gg = ctx.gg if ctx.gg is not None else torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        gb = ctx.gb if ctx.gb is not None else torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        dx = ext().layernorm_bwd(dy.contiguous(), x, mean, rstd, g, None, gg, gb)
        return dx, None, None, None, None, None


class _LayerNormResidualFn(torch.autograd.Function):
    """Returns ``(x, LN(x))``.  The first output carries the residual stream past the sub-layer, so the gradients of
    both uses of ``x`` arrive in one backward call and are summed inside the LayerNorm backward kernel instead of by a
    separate element-wise add."""

    @staticmethod
    def forward(ctx, x, g, b, gg, gb, eps):
        y, mean, rstd = ext().layernorm_fwd(x, g, b, eps)
        ctx.save_for_backward(x, mean, rstd, g)
        ctx.gg, ctx.gb = gg, gb
        return x.view_as(x), y

    @staticmethod
    def backward(ctx, dres, dy):
        if dy is None:
            return dres, None, None, None, None, None
        x, mean, rstd, g = ctx.saved_tensors
        gg = ctx.gg if ctx.gg is not None else torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        gb = ctx.gb if ctx.gb is not None else torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        if dres is not None:
            dres = dres.contiguous() if dres.dtype == torch.bfloat16 else dres.to(torch.bfloat16).contiguous()
        dx = ext().layernorm_bwd(dy.contiguous(), x, mean, rstd, g, dres, gg, gb)
        return dx, None, None, None, None, None


def layer_norm_residual(x, weight, bias, eps=1e-5):
    """``(x, LN(x))`` for a pre-norm residual block ``x + f(LN(x))``: pass the first result as the residual."""
    if (fused_param(weight) and x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and x.is_contiguous()
            and x.shape[-1] <= 16384 and x.shape[-1] % 8 == 0 and torch.is_grad_enabled() and x.requires_grad):
        return _LayerNormResidualFn.apply(x, weight.work, bias.work, getattr(weight, "main_grad", None),
                                          getattr(bias, "main_grad", None), eps)
    return x, layer_norm(x, weight, bias, eps)


def layer_norm(x, weight, bias, eps=1e-5):
    if fused_param(weight) and x.is_cuda and x.shape[-1] <= 16384 and x.shape[-1] % 8 == 0:
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
            y = _LayerNormFn.apply(_track(x2), weight.work, bias.work, getattr(weight, "main_grad", None),
                                   getattr(bias, "main_grad", None), eps)
        else:
            y = ext().layernorm_fwd(x2, weight.work, bias.work, eps)[0]
        return y.reshape(shp)
    return ref.layer_norm(x, weight, bias, eps)


# ---------------------------------------------------------------------------------------------------
# attention over packed sequences
# ---------------------------------------------------------------------------------------------------
class _AttnFn(torch.autograd.Function):
    """Packed attention over fused projections.

    ``a`` is either the fused self-attention projection ``[N, 3*W]`` (``b`` is None) or the query projection
    ``[Nq, W]`` with ``b`` the fused key/value projection ``[Nk, 2*W]``.  Gradients come back in the same
    fused layouts, so no slice-scatter kernels run in backward.
    """

    @staticmethod
    def forward(ctx, a, b, cu_q, cu_k, heads, max_q, max_k, causal, scale, p, seed, sid):
        W = heads * 64
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
        else:
            q, k, v = a, b[:, :W], b[:, W:]
        out = torch.empty((q.shape[0], W), dtype=torch.bfloat16, device=q.device)   # the kernel clears rows past the last sequence
        lse = torch.empty((heads, q.shape[0]), dtype=torch.float32, device=q.device)
        ext().attn_fwd(q, k, v, out, lse, cu_q, cu_k, heads, max_q, max_k, causal, scale, p, seed, sid)
        ctx.save_for_backward(a, b, out, lse, cu_q, cu_k)
        ctx.cfg = (heads, max_q, max_k, causal, scale, p, seed, sid)
        return out

    @staticmethod
    def backward(ctx, d_out):
        a, b, out, lse, cu_q, cu_k = ctx.saved_tensors
        heads, max_q, max_k, causal, scale, p, seed, sid = ctx.cfg
        W = heads * 64
        da = torch.empty_like(a)        # every sequence row is written by the kernel, the rest is cleared by it
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
            dq, dk, dv = da[:, :W], da[:, W:2 * W], da[:, 2 * W:]
            db = None
        else:
            db = torch.empty_like(b)
            q, k, v = a, b[:, :W], b[:, W:]
            dq, dk, dv = da, db[:, :W], db[:, W:]
        dq_acc = torch.zeros((q.shape[0], W), dtype=torch.float32, device=q.device) if max_k > 128 else None
        ext().attn_bwd(q, k, v, out, lse, d_out.contiguous(), dq, dk, dv, dq_acc, cu_q, cu_k, heads, max_q, max_k, causal,
                       scale, p, seed, sid)
        return (da, db) + (None,) * 10


class _AttnBiasFn(torch.autograd.Function):
    """``_AttnFn`` with an additive fp32 score bias ``[batch, heads, max_q, max_k]`` (relative-position terms): the bias is
    added to the scaled scores inside the kernels, its gradient (dS before the softmax scale) comes back in the same
    layout.  Always the general multi-tile kernels."""

    @staticmethod
    def forward(ctx, a, b, bias, cu_q, cu_k, heads, max_q, max_k, causal, scale, p, seed, sid):
        W = heads * 64
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
        else:
            q, k, v = a, b[:, :W], b[:, W:]
        out = torch.empty((q.shape[0], W), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((heads, q.shape[0]), dtype=torch.float32, device=q.device)
        ext().attn_fwd_bias(q, k, v, out, lse, cu_q, cu_k, heads, max_q, max_k, causal, scale, p, seed, sid, bias)
        LAUNCHES[0] += 1
        ctx.save_for_backward(a, b, bias, out, lse, cu_q, cu_k)
        ctx.cfg = (heads, max_q, max_k, causal, scale, p, seed, sid)
        return out

    @staticmethod
    def backward(ctx, d_out):
        a, b, bias, out, lse, cu_q, cu_k = ctx.saved_tensors
        heads, max_q, max_k, causal, scale, p, seed, sid = ctx.cfg
        W = heads * 64
        da = torch.empty_like(a)
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
            dq, dk, dv = da[:, :W], da[:, W:2 * W], da[:, 2 * W:]
            db = None
        else:
            db = torch.empty_like(b)
            q, k, v = a, b[:, :W], b[:, W:]
            dq, dk, dv = da, db[:, :W], db[:, W:]
        dq_acc = torch.zeros((q.shape[0], W), dtype=torch.float32, device=q.device) if max_k > 128 else None
        # same strides as the bias (it may be a padded view); pairs outside the sequences stay zero
        dbias = (torch.empty_strided(bias.shape, bias.stride(), dtype=bias.dtype, device=bias.device).zero_()
                 if ctx.needs_input_grad[2] else None)
        ext().attn_bwd_bias(q, k, v, out, lse, d_out.contiguous(), dq, dk, dv, dq_acc, cu_q, cu_k, heads, max_q, max_k, causal,
                            scale, p, seed, sid, bias, dbias)
        LAUNCHES[0] += 1
        return (da, db, dbias) + (None,) * 10


def _attn_dispatch(a, b, cu_q, cu_k, heads, max_q, max_k, causal, dropout_p, training, scale, bias=None):
    W = (a.shape[1] // 3) if b is None else a.shape[1]
    d = W // heads
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    p = float(dropout_p) if training else 0.0
    if a.is_cuda and a.dtype == torch.bfloat16 and d < 64 and d % 8 == 0:
        # heads narrower than the kernels' 64 columns: zero columns change neither q . k nor the first d output columns
        n = a.shape[0]

        def widen(t, parts):
            return F.pad(t.reshape(t.shape[0], parts, heads, d), (0, 64 - d)).reshape(t.shape[0], parts * heads * 64)

        out = _attn_dispatch(widen(a, 3 if b is None else 1), None if b is None else widen(b, 2), cu_q, cu_k, heads, max_q, max_k,
                             causal, dropout_p, training, scale, bias)
        return out.view(n, heads, 64)[..., :d].reshape(n, heads * d)
    if bias is not None and a.is_cuda and d == 64 and a.dtype == torch.bfloat16:
        sid = next_stream() if p > 0 else 0
        a = a.contiguous()
        b = b.contiguous() if b is not None else None
        bias = bias.float()
        if bias.stride(-1) != 1:
            bias = bias.contiguous()
        if not torch.is_grad_enabled():
            bias = bias.detach()
        return _AttnBiasFn.apply(a, b, bias, cu_q, cu_k, heads, int(max_q), int(max_k), bool(causal), scale, p, _Rng.seed, sid)
    if bias is not None:
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
        else:
            q, k, v = a, b[:, :W], b[:, W:]
        return ref.attention(q, k, v, cu_q, cu_k, heads, causal, p, scale, bias=bias)
    if a.is_cuda and d == 64 and a.dtype == torch.bfloat16:
        sid = next_stream() if p > 0 else 0
        a = a.contiguous()
        b = b.contiguous() if b is not None else None
        if torch.is_grad_enabled() and (a.requires_grad or (b is not None and b.requires_grad)):
            return _AttnFn.apply(a, b, cu_q, cu_k, heads, int(max_q), int(max_k), bool(causal), scale, p, _Rng.seed, sid)
        if b is None:
            q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
        else:
            q, k, v = a, b[:, :W], b[:, W:]
        out = torch.empty((q.shape[0], W), dtype=torch.bfloat16, device=q.device)   # the kernel clears rows past the last sequence
        lse = torch.empty((heads, q.shape[0]), dtype=torch.float32, device=q.device)
        ext().attn_fwd(q, k, v, out, lse, cu_q, cu_k, heads, int(max_q), int(max_k), bool(causal), scale, p, _Rng.seed, sid)
        return out
    if b is None:
        q, k, v = a[:, :W], a[:, W:2 * W], a[:, 2 * W:]
    else:
        q, k, v = a, b[:, :W], b[:, W:]
    return ref.attention(q, k, v, cu_q, cu_k, heads, causal, p, scale)


def self_attention(qkv, cu, heads, max_len, causal=False, dropout_p=0.0, training=True, scale=None, bias=None):
    """Packed self-attention on the fused projection ``qkv [N, 3*heads*d]`` (columns = [q | k | v]).  ``bias``: optional
    additive term ``[batch, heads, >= max_len, >= max_len]`` on the scaled scores (entry ``[b, h, i, j]`` belongs to query
    ``i`` and key ``j`` of sequence ``b``); differentiable."""
    return _attn_dispatch(qkv, None, cu, cu, heads, max_len, max_len, causal, dropout_p, training, scale, bias)


def cross_attention(q, kv, cu_q, cu_k, heads, max_q, max_k, dropout_p=0.0, training=True, scale=None, bias=None):
    """Packed encoder-decoder attention: ``q [Nq, heads*d]``, fused ``kv [Nk, 2*heads*d]`` (columns = [k | v])."""
    return _attn_dispatch(q, kv, cu_q, cu_k, heads, max_q, max_k, False, dropout_p, training, scale, bias)


def attention(q, k, v, cu_q, cu_k, heads, max_q, max_k, causal=False, dropout_p=0.0, training=True, scale=None):
    """Packed attention on separate q / k / v matrices (inference and tests; no autograd on the fused path)."""
    d = q.shape[1] // heads
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    p = float(dropout_p) if training else 0.0
    if q.is_cuda and d == 64 and q.dtype == torch.bfloat16 and not (torch.is_grad_enabled() and q.requires_grad):
        sid = next_stream() if p > 0 else 0
        out = torch.empty((q.shape[0], heads * 64), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((heads, q.shape[0]), dtype=torch.float32, device=q.device)
        ext().attn_fwd(q, k, v, out, lse, cu_q, cu_k, heads, int(max_q), int(max_k), bool(causal), scale, p, _Rng.seed, sid)
        return out
    return ref.attention(q, k, v, cu_q, cu_k, heads, causal, p, scale)


# ---------------------------------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------------------------------
class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dummy, tokens, positions, table, pos_table, gtable, gpos, scale, p, seed, sid, pad_idx):
        out = ext().embed_fwd(tokens, positions, table, pos_table, scale, p, seed, sid)
        ctx.save_for_backward(tokens, positions)
        ctx.cfg = (scale, p, seed, sid, pad_idx)
        ctx.gtable, ctx.gpos = gtable, gpos
        return out

    @staticmethod
    def backward(ctx, dy):
        tokens, positions = ctx.saved_tensors
        scale, p, seed, sid, pad_idx = ctx.cfg
        if ctx.gtable is not None:
            ext().embed_bwd(tokens, positions, dy.contiguous(), ctx.gtable, ctx.gpos, scale, p, seed, sid, pad_idx)
        return (None,) * 12


_dummy = {}


def _grad_anchor(device):
    t = _dummy.get(device)
    if t is None:
        t = torch.zeros(1, device=device, requires_grad=True)
        _dummy[device] = t
    return t


def embedding(tokens, table, positions=None, pos_table=None, scale=1.0, dropout_p=0.0, training=True, pad_idx=0,
              pos_trainable=False):
    """out = dropout(table[tokens] * scale + pos_table[positions]) for 1-D packed ``tokens``."""
    p = float(dropout_p) if training else 0.0
    if fused_param(table) and tokens.is_cuda and table.shape[1] % 16 == 0:
        sid = next_stream() if p > 0 else 0
        pt = None
        gpos = None
        if pos_table is not None:
            pt = pos_table.work if fused_param(pos_table) else pos_table
            if pt.dtype != torch.bfloat16:
                pt = pt.to(torch.bfloat16)
            if pos_trainable and fused_param(pos_table) and pos_table.requires_grad:
                gpos = pos_table.main_grad
        gtable = table.main_grad if table.requires_grad else None
        if torch.is_grad_enabled() and (gtable is not None or gpos is not None):
            return _EmbedFn.apply(_grad_anchor(tokens.device), tokens, positions, table.work, pt, gtable, gpos, scale, p,
                                  _Rng.seed, sid, pad_idx)
        return ext().embed_fwd(tokens, positions, table.work, pt, scale, p, _Rng.seed, sid)
    return ref.embedding(tokens, table, positions, pos_table, scale, p, pad_idx)


# ---------------------------------------------------------------------------------------------------
# dropout + residual
# ---------------------------------------------------------------------------------------------------
class _DropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, seed, sid):
        ctx.cfg = (p, seed, sid, residual is not None)
        return ext().dropout_add(x, residual, p, seed, sid)

    @staticmethod
    def backward(ctx, dy):
        p, seed, sid, has_res = ctx.cfg
        dy = dy.contiguous()
        dx = ext().dropout_add(dy, None, p, seed, sid)
        return dx, (dy if has_res else None), None, None, None


def dropout_add(x, residual=None, p=0.0, training=True):
    """``residual + dropout(x)`` (``residual`` optional)."""
    p = float(p) if training else 0.0
    if x.is_cuda and x.dtype == torch.bfloat16 and extension_available() and x.numel() % 16 == 0 and p > 0:
        return _DropoutAddFn.apply(x.contiguous(), residual.contiguous() if residual is not None else None, p, _Rng.seed,
                                   next_stream())
    return ref.dropout_add(x, residual, p)


# ---------------------------------------------------------------------------------------------------
# label-smoothed cross-entropy
# ---------------------------------------------------------------------------------------------------
class _XentFn(torch.autograd.Function):
    """Forward computes the loss AND overwrites the logits with d(loss_sum)/d(logits); backward scales."""

    @staticmethod
    def forward(ctx, logits, labels, smoothing, pad_idx):
        loss_sum = torch.zeros(1, dtype=torch.float32, device=logits.device)
        correct = torch.zeros(1, dtype=torch.float32, device=logits.device)
        row_loss = ext().xent_fused(logits, labels, smoothing, pad_idx, loss_sum, correct, None, 1.0, True)
        ctx.save_for_backward(logits)
        ctx.mark_non_differentiable(correct, row_loss)
        return loss_sum, correct, row_loss

    @staticmethod
    def backward(ctx, g_loss, _g1, _g2):
        (dlogits,) = ctx.saved_tensors
        # the common case is g_loss == 1 (or a constant loss scale): scale lazily
        return dlogits * g_loss.to(dlogits.dtype), None, None, None


def cross_entropy(logits, labels, smoothing=0.0, pad_idx=0):
    """Summed label-smoothed CE over non-pad rows.  Returns (loss_sum[1], n_correct[1], row_loss[rows]).

    On the fused path ``logits`` (bf16, 2-D) is consumed: its storage is overwritten with the gradient.
    """
    if logits.is_cuda and logits.dtype == torch.bfloat16 and extension_available() and logits.stride(0) % 8 == 0 and logits.stride(1) == 1:
        labels = labels.contiguous()
        if torch.is_grad_enabled() and logits.requires_grad:
            return _XentFn.apply(logits, labels, float(smoothing), int(pad_idx))
        loss_sum = torch.zeros(1, dtype=torch.float32, device=logits.device)
        correct = torch.zeros(1, dtype=torch.float32, device=logits.device)
        row_loss = ext().xent_fused(logits, labels, float(smoothing), int(pad_idx), loss_sum, correct, None, 1.0, False)
        return loss_sum, correct, row_loss
    return ref.cross_entropy(logits, labels, smoothing, pad_idx)


class _GeneratorXentFn(torch.autograd.Function):
    """logits = h W^T (+b) -> fused CE -> dh, dW in one autograd node.

    The [rows, V] logits buffer is overwritten in place with its own gradient, already multiplied by
    ``grad_scale`` (a float or a 1-element device tensor read by the kernel, so no host round trip).  The
    upstream gradient of ``loss_sum`` is therefore taken to be 1 when ``grad_scale`` is given.
    """

    @staticmethod
    def forward(ctx, h, w, bias, gw, gb, labels, smoothing, pad_idx, grad_scale):
        rows, V = h.shape[0], w.shape[0]
        logits = empty_rows(rows, V, h.device)
        gemm(h, w, logits, bias=bias)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=h.device)
        correct = torch.zeros(1, dtype=torch.float32, device=h.device)
        gs_t = grad_scale if isinstance(grad_scale, torch.Tensor) else None
        gs_v = 1.0 if (grad_scale is None or gs_t is not None) else float(grad_scale)
        row_loss = ext().xent_fused(logits, labels, smoothing, pad_idx, loss_sum, correct, gs_t, gs_v, True)
        ctx.save_for_backward(h, w, logits)
        ctx.gw, ctx.gb = gw, gb
        ctx.prescaled = grad_scale is not None
        ctx.mark_non_differentiable(correct, row_loss)
        return loss_sum, correct, row_loss

    @staticmethod
    def backward(ctx, g_loss, _g1, _g2):
        h, w, dlogits = ctx.saved_tensors
        if not ctx.prescaled:
            dlogits = dlogits * g_loss.to(dlogits.dtype)
        dh = torch.empty_like(h)
        gemm(dlogits, w, dh, b_mn_major=True)
        if ctx.gw is not None:
            gemm(dlogits, h, ctx.gw, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
        if ctx.gb is not None:
            ext().colsum(dlogits, ctx.gb)
        return (dh,) + (None,) * 8


class _GeneratorXentChunkedFn(torch.autograd.Function):
    """``_GeneratorXentFn`` without the ``[rows, V]`` buffer: the rows are processed ``chunk`` at a time through one
    ``[chunk, V]`` scratch that stays in L2 between its four uses (logits GEMM -> fused CE in place -> dH GEMM ->
    dW GEMM), so the logits never travel to HBM.  Gradients are produced during the forward call (the CE kernel
    writes them anyway), which is why a ``grad_scale`` must be given: the upstream gradient is taken to be 1."""

    @staticmethod
    def forward(ctx, h, w, bias, gw, gb, labels, smoothing, pad_idx, grad_scale, chunk):
        rows, V = h.shape[0], w.shape[0]
        scratch = empty_rows(chunk, V, h.device)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=h.device)
        correct = torch.zeros(1, dtype=torch.float32, device=h.device)
        gs_t = grad_scale if isinstance(grad_scale, torch.Tensor) else None
        gs_v = 1.0 if gs_t is not None else float(grad_scale)
        dh = torch.empty_like(h)
        row_losses = []
        for r0 in range(0, rows, chunk):
            r1 = min(r0 + chunk, rows)
            lg = scratch[:r1 - r0]
            gemm(h[r0:r1], w, lg, bias=bias)
            row_losses.append(ext().xent_fused(lg, labels[r0:r1], smoothing, pad_idx, loss_sum, correct, gs_t, gs_v, True))
            gemm(lg, w, dh[r0:r1], b_mn_major=True)
            if gw is not None:
                gemm(lg, h[r0:r1], gw, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
            if gb is not None:
                ext().colsum(lg, gb)
        row_loss = torch.cat(row_losses) if len(row_losses) > 1 else row_losses[0]
        ctx.save_for_backward(dh)
        ctx.mark_non_differentiable(correct, row_loss)
        return loss_sum, correct, row_loss

    @staticmethod
    def backward(ctx, g_loss, _g1, _g2):
        (dh,) = ctx.saved_tensors
        return (dh,) + (None,) * 9


def generator_cross_entropy(h, weight, bias, labels, smoothing=0.0, pad_idx=0, grad_scale=None, chunk_rows: int = 0):
    """Output projection + label-smoothed CE.  Returns (loss_sum, n_correct, row_loss).  ``chunk_rows`` > 0 (with a
    ``grad_scale``) selects the chunked variant that keeps the logits out of HBM."""
    if fused_param(weight) and h.is_cuda:
        b = bias.work if bias is not None else None
        gw = weight.main_grad if weight.requires_grad else None
        gb = bias.main_grad if (bias is not None and bias.requires_grad) else None
        hin = (h if h.dtype == torch.bfloat16 else h.to(torch.bfloat16)).contiguous()
        if torch.is_grad_enabled() and chunk_rows > 0 and grad_scale is not None and h.shape[0] > chunk_rows:
            return _GeneratorXentChunkedFn.apply(_track(hin), weight.work, b, gw, gb, labels.contiguous(), float(smoothing),
                                                 int(pad_idx), grad_scale, int(chunk_rows))
        if torch.is_grad_enabled():
            return _GeneratorXentFn.apply(_track(hin), weight.work, b, gw, gb, labels.contiguous(), float(smoothing), int(pad_idx),
                                          grad_scale)
        logits = empty_rows(h.shape[0], weight.shape[0], h.device)
        gemm(hin, weight.work, logits, bias=b)
        return cross_entropy(logits, labels, smoothing, pad_idx)
    logits = ref.linear(h, weight, bias, 0, 0.0, None)
    loss_sum, correct, row_loss = ref.cross_entropy(logits, labels, smoothing, pad_idx)
    if grad_scale is not None and torch.is_grad_enabled():
        # same contract as the fused path: backward of loss_sum yields grad_scale-scaled gradients
        gs = grad_scale if isinstance(grad_scale, torch.Tensor) else torch.tensor(float(grad_scale))
        loss_sum = ref.scale_gradient(loss_sum, gs.to(loss_sum.device))
    return loss_sum, correct, row_loss

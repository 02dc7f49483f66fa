"""Per-kernel micro-benchmarks on the shapes of the Transformer-big training step.

    python -m nmtgminor_b200.ops.bench_kernels [--json out.json] [--only gemm,attn,attn_long,...]   (--only gemm_stalls: cycle breakdown of the CTA-pair GEMM)

Each kernel is timed with CUDA events after warm-up; between timed launches a 256 MB buffer is rewritten so
the 126 MB L2 starts cold.  GEMMs report TFLOP/s next to ``torch.matmul`` (cuBLAS) on the same shape as a
yardstick; memory-bound kernels report GB/s of their algorithmic traffic.  When ``MEASURED_PEAKS.json`` sits
at the repository root the fractions "of measured" peak are printed as well.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .. import ops

_FLUSH = None


def _flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.add_(1)


def time_ms(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            _flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "fallback"


def bench_gemm(rows):
    T, H, F, V = 8192, 1024, 4096, 32000
    dev = "cuda"
    shapes = [
        ("qkv fwd", T, 3 * H, H, False, False, "bf16"), ("out fwd", T, H, H, False, False, "bf16"),
        ("fc1 fwd", T, F, H, False, False, "bf16"), ("fc2 fwd", T, H, F, False, False, "bf16"),
        ("generator fwd", T, V, H, False, False, "bf16"),
        ("fc1 dgrad", T, H, F, False, True, "bf16"), ("fc2 dgrad", T, F, H, False, True, "bf16"),
        ("qkv dgrad", T, H, 3 * H, False, True, "bf16"), ("generator dgrad", T, H, V, False, True, "bf16"),
        ("fc1 wgrad", F, H, T, True, True, "fp32"), ("fc2 wgrad", H, F, T, True, True, "fp32"),
        ("out wgrad", H, H, T, True, True, "fp32"), ("qkv wgrad", 3 * H, H, T, True, True, "fp32"),
        ("generator wgrad", V, H, T, True, True, "fp32"),
    ]
    for name, M, N, K, a_mn, b_mn, odt in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
        out = torch.zeros(M, N, device=dev, dtype=torch.float32 if odt == "fp32" else torch.bfloat16)
        acc = odt == "fp32"
        ms = time_ms(lambda: ops.gemm(a, b, out, a_mn_major=a_mn, b_mn_major=b_mn, accumulate=acc, allow_split_k=acc))
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms_ref = time_ms(lambda: torch.matmul(A, Bt, out=ref))
        fl = 2.0 * M * N * K
        rows.append({"kernel": "gemm " + name, "shape": [M, N, K], "ms": ms, "tflops": fl / ms / 1e9,
                     "cublas_ms": ms_ref, "cublas_tflops": fl / ms_ref / 1e9})


def bench_mlp_epilogues(rows):
    T, H, F = 8192, 1024, 4096
    x = torch.randn(T, H, device="cuda").bfloat16()
    w1 = torch.randn(F, H, device="cuda").bfloat16()
    b1 = torch.randn(F, device="cuda").bfloat16()
    h = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(T, H, device="cuda").bfloat16()
    w2 = torch.randn(H, F, device="cuda").bfloat16()
    b2 = torch.randn(H, device="cuda").bfloat16()
    y = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * T * H * F
    ms = time_ms(lambda: ops.gemm(x, w1, h, bias=b1, act=1, dropout_p=0.1, seed=1, stream_id=1))
    rows.append({"kernel": "gemm fc1 + bias + relu + dropout", "shape": [T, F, H], "ms": ms, "tflops": fl / ms / 1e9})
    ms = time_ms(lambda: ops.gemm(h, w2, y, bias=b2, residual=res, dropout_p=0.1, seed=1, stream_id=2))
    rows.append({"kernel": "gemm fc2 + bias + dropout + residual", "shape": [T, H, F], "ms": ms, "tflops": fl / ms / 1e9})
    ms = time_ms(lambda: ops.gemm(y, w2, h, b_mn_major=True, aux=h, act=5, alpha=1.1))
    rows.append({"kernel": "gemm fc2 dgrad + relu' (aux = h)", "shape": [T, F, H], "ms": ms, "tflops": fl / ms / 1e9})
    bits = torch.empty(T, F // 32, dtype=torch.int32, device="cuda")
    ms = time_ms(lambda: ops.gemm(x, w1, h, bias=b1, act=1, dropout_p=0.1, seed=1, stream_id=1, mask=bits))
    rows.append({"kernel": "gemm fc1 + bias + relu + dropout + sign bits", "shape": [T, F, H], "ms": ms, "tflops": fl / ms / 1e9})
    dz = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    ms = time_ms(lambda: ops.gemm(y, w2, dz, b_mn_major=True, act=8, mask=bits, alpha=1.1))
    rows.append({"kernel": "gemm fc2 dgrad + relu' (sign bits)", "shape": [T, F, H], "ms": ms, "tflops": fl / ms / 1e9})


def bench_elementwise(rows):
    T, H, V = 8192, 1024, 32000
    e = ops.ext()
    x = torch.randn(T, H, device="cuda").bfloat16()
    g = torch.ones(H, device="cuda").bfloat16()
    b = torch.zeros(H, device="cuda").bfloat16()
    ms = time_ms(lambda: e.layernorm_fwd(x, g, b, 1e-5))
    rows.append({"kernel": "layernorm fwd", "shape": [T, H], "ms": ms, "gbs": 2 * T * H * 2 / ms / 1e6})
    y, mean, rstd = e.layernorm_fwd(x, g, b, 1e-5)
    dg, db = torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda")
    ms = time_ms(lambda: e.layernorm_bwd(x, x, mean, rstd, g, x, dg, db))
    rows.append({"kernel": "layernorm bwd (+residual grad)", "shape": [T, H], "ms": ms, "gbs": 4 * T * H * 2 / ms / 1e6})
    ms = time_ms(lambda: e.dropout_add(x, x, 0.1, 1, 1))
    rows.append({"kernel": "dropout_add", "shape": [T, H], "ms": ms, "gbs": 3 * T * H * 2 / ms / 1e6})
    logits = torch.randn(T, V, device="cuda").bfloat16()
    labels = torch.randint(1, V, (T,), device="cuda")
    ls = torch.zeros(1, device="cuda")
    ms = time_ms(lambda: e.xent_fused(logits, labels, 0.1, 0, ls, None, None, 1.0, True), iters=5)
    rows.append({"kernel": "xent fwd+bwd fused", "shape": [T, V], "ms": ms, "gbs": 2 * T * V * 2 / ms / 1e6})
    n = 209_087_744 // 4 * 4
    master, grad, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    work = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    master.normal_(0, 0.02), grad.normal_(0, 1e-3), m.normal_(0, 1e-4), v.uniform_(0, 1e-6)
    hyper = torch.zeros(16)
    hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], hyper[7], hyper[8] = 1e-3, 0.9, 0.997, 1e-9, 0.01, 0.1, 0.003, 1.0, 5.0
    hyper.view(torch.int32)[9:11] = 1          # decoupled weight decay, clear the gradients: what the training step runs
    hyper = hyper.cuda()
    sq = torch.zeros(1, device="cuda")
    bad = torch.zeros(1, device="cuda", dtype=torch.int32)
    ms = time_ms(lambda: e.sq_norm(grad, sq, bad), iters=5)
    rows.append({"kernel": "grad sq-norm (209M)", "shape": [n], "ms": ms, "gbs": n * 4 / ms / 1e6})
    ms = time_ms(lambda: e.adamw_flat(master, work, grad, m, v, hyper, sq, bad), iters=5)
    rows.append({"kernel": "adamw flat (209M)", "shape": [n], "ms": ms, "gbs": n * (4 * 4 + 4 * 4 + 2) / ms / 1e6})   # reads p, g, m, v; writes p, g, m, v, bf16 p


def bench_attention(rows):
    import numpy as np
    rng = np.random.RandomState(0)
    lens = []
    while sum(lens) < 8192 - 100:
        lens.append(int(rng.randint(20, 101)))
    n = sum(lens)
    cap = (n + 127) // 128 * 128
    heads, W = 16, 1024
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.cuda()
    qkv = torch.randn(cap, 3 * W, device="cuda").bfloat16()
    out = torch.zeros(cap, W, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(heads, cap, device="cuda")
    e = ops.ext()
    q, k, v = qkv[:, :W], qkv[:, W:2 * W], qkv[:, 2 * W:]
    for causal in (False, True):
        ms = time_ms(lambda: e.attn_fwd(q, k, v, out, lse, cu, cu, heads, 100, 100, causal, 0.125, 0.1, 1, 1))
        fl = sum(4.0 * L * L * 64 * heads for L in lens)
        rows.append({"kernel": "attention fwd causal=%s (%d seqs, %d tokens)" % (causal, len(lens), n), "ms": ms,
                     "tflops": fl / ms / 1e9})
        dqkv = torch.zeros_like(qkv)
        dout = torch.randn_like(out)
        ms = time_ms(lambda: e.attn_bwd(q, k, v, out, lse, dout, dqkv[:, :W], dqkv[:, W:2 * W], dqkv[:, 2 * W:], None, cu, cu,
                                        heads, 100, 100, causal, 0.125, 0.1, 1, 1))
        rows.append({"kernel": "attention bwd causal=%s" % causal, "ms": ms, "tflops": 2.5 * fl / ms / 1e9})


def bench_attention_ablation(rows):
    """Short-sequence attention backward with parts of the work switched off (every barrier hand-shake kept): which role
    bounds the item rate.  Same workload as ``bench_attention``."""
    import numpy as np
    rng = np.random.RandomState(0)
    lens = []
    while sum(lens) < 8192 - 100:
        lens.append(int(rng.randint(20, 101)))
    n = sum(lens)
    cap = (n + 127) // 128 * 128
    heads, W = 16, 1024
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.cuda()
    qkv = torch.randn(cap, 3 * W, device="cuda").bfloat16()
    out = torch.zeros(cap, W, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(heads, cap, device="cuda")
    e = ops.ext()
    q, k, v = qkv[:, :W], qkv[:, W:2 * W], qkv[:, 2 * W:]
    e.attn_fwd(q, k, v, out, lse, cu, cu, heads, 100, 100, False, 0.125, 0.1, 1, 1)
    dqkv = torch.zeros_like(qkv)
    dout = torch.randn_like(out)
    names = {0: "everything", 1: "no P/dS math", 2: "no gradient read-out", 4: "no gradient MMAs", 8: "no S/dP MMAs", 16: "no TMA loads",
             32: "no D / log-sum-exp loads", 64: "no dropout masks", 3: "no math, no read-out", 19: "no math, no read-out, no loads",
             31: "barriers only", 12: "no MMAs"}
    try:
        for bits, name in names.items():
            e.set_attn_bwd_ablation(bits)
            ms = time_ms(lambda: e.attn_bwd(q, k, v, out, lse, dout, dqkv[:, :W], dqkv[:, W:2 * W], dqkv[:, 2 * W:], None, cu, cu,
                                            heads, 100, 100, False, 0.125, 0.1, 1, 1))
            rows.append({"kernel": "attention bwd short, %s" % name, "ms": ms, "items_per_cta": len(lens) * heads / 148.0})
    finally:
        e.set_attn_bwd_ablation(0)


def bench_attention_long_ablation(rows):
    """The pipelined multi-tile backward (8 x 1500 frames, 20 heads) with parts of the work switched off, every barrier
    hand-shake kept: which role bounds the tile rate."""
    e = ops.ext()
    L, heads, B = 1500, 20, 8
    W = heads * 64
    n = B * L
    cu = (torch.arange(B + 1, dtype=torch.int32) * L).cuda()
    qkv = torch.randn(n, 3 * W, device="cuda").bfloat16()
    q, k, v = qkv[:, :W], qkv[:, W:2 * W], qkv[:, 2 * W:]
    out = torch.empty(n, W, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(heads, n, device="cuda")
    e.attn_fwd(q, k, v, out, lse, cu, cu, heads, L, L, False, 0.125, 0.0, 1, 0)
    dqkv = torch.empty_like(qkv)
    dq_acc = torch.empty(n, W, device="cuda", dtype=torch.float32)
    dout = torch.randn_like(out)
    names = {0: "everything", 1: "no P/dS math", 2: "no dQ read-out", 32: "dQ staged, not added", 4: "no gradient MMAs", 8: "no S/dP MMAs",
             12: "no MMAs", 3: "no math, no read-out", 15: "barriers only"}
    try:
        for bits, name in names.items():
            e.set_attn_bwd_ablation(bits)

            def run():
                dq_acc.zero_()
                e.attn_bwd(q, k, v, out, lse, dout, dqkv[:, :W], dqkv[:, W:2 * W], dqkv[:, 2 * W:], dq_acc, cu, cu, heads, L, L, False,
                           0.125, 0.0, 1, 0)
            rows.append({"kernel": "attention bwd 8 x 1500 pipelined, %s" % name, "ms": time_ms(run)})
        rows.append({"kernel": "attention fwd 8 x 1500 pipelined",
                     "ms": time_ms(lambda: e.attn_fwd(q, k, v, out, lse, cu, cu, heads, L, L, False, 0.125, 0.0, 1, 0))})
        # time lines of the first CTA (SM clocks relative to its first stamp), one row per key / query tile
        e.set_attn_bwd_ablation(128)
        e.attn_fwd(q, k, v, out, lse, cu, cu, heads, L, L, False, 0.125, 0.0, 1, 0)
        torch.cuda.synchronize()
        tr = e.attn_fws_trace()[:12]
        t0 = int(tr[tr > 0].min())
        names = ["S rdy", "loaded", "max", "exps", "packed", "pv done", "staged", "PV0 seen", "iss S0", "iss PV0", "iss S1", "iss PV1", "PV0 beg", "PV0 end",
                 "S0 beg", "S0 end"]
        print("forward, CTA 0 (SM clocks):     " + " ".join("%8s" % n for n in names))
        for i in range(12):
            print("  key tile %2d                  " % i + " ".join("%8d" % (int(v) - t0 if int(v) > 0 else -1) for v in tr[i][:16]))
        run()
        torch.cuda.synchronize()
        tr = e.attn_ws_trace()[:12]
        t0 = int(tr[tr > 0].min())
        names = ["Slo rdy", "Slo ld", "lo cmp", "lo st", "Shi rdy", "Shi ld", "hi cmp", "hi st", "iss Slo", "iss Shi", "iss G", "G done",
                 "dQ stg", "dQ out", "TMA iss"]
        print("time line of CTA 0 (SM clocks): " + " ".join("%8s" % n for n in names))
        for i in range(12):
            print("  tile %2d                      " % i + " ".join("%8d" % (int(v) - t0 if int(v) > 0 else -1) for v in tr[i][:15]))
    finally:
        e.set_attn_bwd_ablation(0)


def bench_attention_long(rows):
    """The general multi-tile kernels on speech-length sequences: 8 x 1500 encoder frames with 20 heads (Whisper-large
    encoder self-attention, no dropout) and 8 x 448 causal with dropout 0.1 (decoder self-attention)."""
    e = ops.ext()
    for L, heads, causal, p in ((1500, 20, False, 0.0), (448, 20, True, 0.1), (1000, 16, False, 0.1)):
        B, W = 8, heads * 64
        n = B * L
        cap = (n + 127) // 128 * 128
        cu = (torch.arange(B + 1, dtype=torch.int32) * L).cuda()
        qkv = torch.randn(cap, 3 * W, device="cuda").bfloat16()
        out = torch.zeros(cap, W, device="cuda", dtype=torch.bfloat16)
        lse = torch.empty(heads, cap, device="cuda")
        q, k, v = qkv[:, :W], qkv[:, W:2 * W], qkv[:, 2 * W:]
        fl = 4.0 * L * L * 64 * heads * B * (0.5 if causal else 1.0)
        ms = time_ms(lambda: e.attn_fwd(q, k, v, out, lse, cu, cu, heads, L, L, causal, 0.125, p, 1, 1))
        rows.append({"kernel": "attention fwd %d x %d, %d heads, causal=%s, p=%.1f" % (B, L, heads, causal, p), "ms": ms,
                     "tflops": fl / ms / 1e9})
        dqkv = torch.zeros_like(qkv)
        dout = torch.randn_like(out)
        acc = torch.zeros(cap, W, device="cuda")

        def bwd():
            acc.zero_()
            e.attn_bwd(q, k, v, out, lse, dout, dqkv[:, :W], dqkv[:, W:2 * W], dqkv[:, 2 * W:], acc, cu, cu, heads, L, L,
                       causal, 0.125, p, 1, 1)
        ms = time_ms(bwd)
        rows.append({"kernel": "attention bwd (incl. clearing the dQ accumulator)", "ms": ms, "tflops": 2.5 * fl / ms / 1e9})
        # the kernels without warp specialisation (one role per CTA), for comparison
        e.set_attention_variant(2)
        try:
            ms = time_ms(lambda: e.attn_fwd(q, k, v, out, lse, cu, cu, heads, L, L, causal, 0.125, p, 1, 1))
            rows.append({"kernel": "  fwd, kernel without warp specialisation", "ms": ms, "tflops": fl / ms / 1e9})
            ms = time_ms(bwd)
            rows.append({"kernel": "  bwd, kernel without warp specialisation", "ms": ms, "tflops": 2.5 * fl / ms / 1e9})
        finally:
            e.set_attention_variant(0)
        # the library kernels on the same problem (padded [B, H, L, 64] layout, which favours them: no packing work)
        import torch.nn.functional as F
        qs, ks, vs = (torch.randn(B, heads, L, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
        ms = time_ms(lambda: F.scaled_dot_product_attention(qs, ks, vs, dropout_p=p, is_causal=causal))
        rows.append({"kernel": "  torch SDPA fwd, same shape", "ms": ms, "tflops": fl / ms / 1e9})
        o = F.scaled_dot_product_attention(qs, ks, vs, dropout_p=p, is_causal=causal)
        go = torch.randn_like(o)
        ms = time_ms(lambda: torch.autograd.grad(o, (qs, ks, vs), go, retain_graph=True))
        rows.append({"kernel": "  torch SDPA bwd, same shape", "ms": ms, "tflops": 2.5 * fl / ms / 1e9})


def bench_gemm_stalls():
    """Where the CTA-pair GEMM spends its cycles: the traced build of the kernel counts, per cluster, how long the MMA
    issuer waited for operands and for a free accumulator and how long the epilogue waited for a finished one; two
    ablations (no epilogue, operand streaming without any MMA) bound what each part could reach alone."""
    T, H, F = 8192, 1024, 4096
    dev = "cuda"
    mk = lambda *shape: torch.randn(*shape, device=dev).bfloat16()
    x, w1, w2, wo, wq = mk(T, H), mk(F, H), mk(H, F), mk(H, H), mk(3 * H, H)
    h = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    y = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    qkv = torch.empty(T, 3 * H, device=dev, dtype=torch.bfloat16)
    b1, b2, res = mk(F), mk(H), mk(T, H)
    bits = torch.empty(T, F // 32, dtype=torch.int32, device=dev)
    gw, gwo = torch.zeros(F, H, device=dev), torch.zeros(H, H, device=dev)
    trace = torch.zeros(16 * 128, dtype=torch.int64, device=dev)
    cases = [
        ("fc1 8192x4096x1024", 2.0 * T * H * F, lambda: ops.gemm(x, w1, h)),
        ("fc1 + bias + relu + dropout + sign bits", 2.0 * T * H * F,
         lambda: ops.gemm(x, w1, h, bias=b1, act=1, dropout_p=0.1, seed=1, stream_id=1, mask=bits)),
        ("fc2 8192x1024x4096", 2.0 * T * H * F, lambda: ops.gemm(h, w2, y)),
        ("fc2 + bias + dropout + residual", 2.0 * T * H * F,
         lambda: ops.gemm(h, w2, y, bias=b2, residual=res, dropout_p=0.1, seed=1, stream_id=2)),
        ("fc2 dgrad + sign bits 8192x4096x1024", 2.0 * T * H * F,
         lambda: ops.gemm(y, w2, h, b_mn_major=True, act=8, mask=bits, alpha=1.1)),
        ("out 8192x1024x1024", 2.0 * T * H * H, lambda: ops.gemm(x, wo, y)),
        ("qkv 8192x3072x1024", 2.0 * T * H * 3 * H, lambda: ops.gemm(x, wq, qkv)),
        ("fc1 wgrad 4096x1024x8192 (fp32 accumulate)", 2.0 * T * H * F,
         lambda: ops.gemm(h, x, gw, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)),
        ("out wgrad 1024x1024x8192 (fp32 accumulate)", 2.0 * T * H * H,
         lambda: ops.gemm(y, x, gwo, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)),
    ]

    def traced(fn):
        ops.ext().set_gemm_trace(trace)
        trace.zero_()
        fn()
        torch.cuda.synchronize()
        ops.ext().set_gemm_trace(None)
        t = trace.view(128, 16).float()
        return t[t[:, 0] > 0].mean(0)

    print("%-44s %9s %8s | %12s %9s %9s %10s | %9s %10s" % ("kernel", "ms", "TFLOP/s", "issuer cyc", "wait acc", "wait ops",
                                                             "first ops", "epi wait", "last epi") + "   per tile: drain / chunks / store issue")
    for name, fl, fn in cases:
        ms = time_ms(fn)              # timed with the production kernel; the traced variant runs once afterwards
        m = traced(fn)
        print("%-44s %9.4f %8.0f | %12.0f %8.1f%% %8.1f%% %10.0f | %8.1f%% %10.0f   %6.0f / %6.0f / %6.0f" % (
            name, ms, fl / ms / 1e9, m[0], 100 * m[1] / m[0], 100 * m[2] / m[0], m[3], 100 * m[5] / m[4], m[6],
            m[8] / m[7], m[9] / m[7], m[10] / m[7]))
    for variant, label in ((12, "no epilogue"), (13, "operand streaming only (no MMA)")):
        ops.ext().set_gemm_variant(variant)
        ops.ext().set_gemm_trace(trace)          # the ablations exist in the traced kernel only
        for name, fl, fn in (cases[0], cases[2], cases[5], cases[7]):
            ms = time_ms(fn)
            trace.zero_()
            fn()
            torch.cuda.synchronize()
            t = trace.view(128, 16).float()
            m = t[t[:, 0] > 0].mean(0)
            print("%-34s %-44s %9.4f ms  %6.0f TFLOP/s-equivalent | issuer %8.0f cyc, waiting for operands %4.1f%%" % (
                label, name, ms, fl / ms / 1e9, m[0], 100 * m[2] / m[0]))
        ops.ext().set_gemm_trace(None)
    ops.ext().set_gemm_variant(10)
    print("kernel status word:", ops.check_status())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default="gemm,mlp,elementwise,attn")
    args = ap.parse_args()
    rows = []
    which = set(args.only.split(","))
    if "gemm_stalls" in which:
        bench_gemm_stalls()
        return
    if "gemm" in which:
        bench_gemm(rows)
    if "mlp" in which:
        bench_mlp_epilogues(rows)
    if "elementwise" in which:
        bench_elementwise(rows)
    if "attn" in which:
        bench_attention(rows)
    if "attn_ablate" in which:
        bench_attention_ablation(rows)
    if "attn_long" in which:
        bench_attention_long(rows)
    if "attn_long_ablate" in which:
        bench_attention_long_ablation(rows)
    tf_peak, bw_peak, kind = peaks()
    for r in rows:
        line = "%-48s %8.3f ms" % (r["kernel"], r["ms"])
        if "tflops" in r:
            line += "  %7.1f TFLOP/s (%.2f of %s bf16 peak)" % (r["tflops"], r["tflops"] / tf_peak, kind)
        if "cublas_tflops" in r:
            line += "   cuBLAS %7.1f TFLOP/s" % r["cublas_tflops"]
        if "gbs" in r:
            line += "  %7.1f GB/s (%.2f of %s HBM peak)" % (r["gbs"], r["gbs"] / bw_peak, kind)
        print(line)
    status = ops.check_status()
    print("kernel status word:", status)
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"rows": rows, "status": status, "peaks": {"bf16_tflops": tf_peak, "hbm_gbs": bw_peak, "kind": kind}}, fh, indent=1)


if __name__ == "__main__":
    main()

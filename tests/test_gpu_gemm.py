"""tcgen05 GEMM against fp32 matmul: operand layouts, ragged shapes, epilogues, split-K."""
import pytest
import torch

from nmtgminor_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[0, 1], ids=["pair", "single"], autouse=True)
def gemm_variant(request):
    """0 = automatic (CTA-pair kernel for M > 128), 1 = single-CTA kernel only."""
    ops.ext().set_gemm_variant(request.param)
    yield request.param
    ops.ext().set_gemm_variant(0)


def _rel_err(got, want):
    got, want = got.float(), want.float()
    return ((got - want).abs().max() / (want.abs().max() + 1e-6)).item()


def _status_ok():
    s = ops.check_status()
    assert s == 0, "kernel status word = %d (a bounded wait timed out)" % s


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 1032, 264), (8192, 1024, 1024), (77, 3072, 1024),
                                   (300, 128, 4096), (4096, 32000, 1024)])
def test_gemm_k_major(M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out)
    torch.cuda.synchronize()
    _status_ok()
    want = a.float() @ b.float().t()
    assert _rel_err(out, want) < 1e-2


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (512, 1024, 640), (1000, 264, 1000), (1024, 4096, 8192)])
def test_gemm_mn_major(a_mn, b_mn, M, N, K):
    torch.manual_seed(1)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_err(out, A.float() @ B.float().t()) < 1e-2


@pytest.mark.parametrize("force_bn", [128, 256])
def test_gemm_tile_widths(force_bn):
    torch.manual_seed(2)
    a = torch.randn(640, 512, device=DEV).bfloat16()
    b = torch.randn(768, 512, device=DEV).bfloat16()
    out = torch.empty(640, 768, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out, force_bn=force_bn)
    _status_ok()
    assert _rel_err(out, a.float() @ b.float().t()) < 1e-2


@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_gemm_bias_act_residual_preact(act):
    torch.manual_seed(3)
    M, N, K = 513, 1024, 256
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = (torch.randn(N, K, device=DEV) / 16).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    res = torch.randn(M, N, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    pre = torch.empty_like(out)
    ops.gemm(a, b, out, bias=bias, residual=res, preact=pre, act=act)
    _status_ok()
    z = a.float() @ b.float().t() + bias.float()
    f = [lambda t: t, torch.relu, torch.nn.functional.gelu, torch.nn.functional.silu][act]
    assert _rel_err(pre, z) < 1e-2
    assert _rel_err(out, f(z) + res.float()) < 1.5e-2


def test_gemm_dropout_epilogue_matches_dropout_kernel():
    torch.manual_seed(4)
    M, N, K = 256, 512, 128
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    plain = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    dropped = torch.empty_like(plain)
    ops.gemm(a, b, plain)
    ops.gemm(a, b, dropped, dropout_p=0.25, seed=99, stream_id=3)
    same_mask = ops.ext().dropout_add(plain, None, 0.25, 99, 3)
    _status_ok()
    assert _rel_err(dropped, same_mask) < 1e-2
    frac = (dropped == 0).float().mean().item()
    assert abs(frac - 0.25) < 0.02


@pytest.mark.parametrize("act,name", [(5, "relu"), (6, "gelu"), (7, "silu")])
def test_gemm_activation_backward_epilogue(act, name):
    torch.manual_seed(5)
    M, N, K = 384, 1024, 256
    dy = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(K, N, device=DEV) / 16).bfloat16()     # dgrad: dh = dy @ w  (w stored [K_red, N])
    aux = torch.randn(M, N, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(dy, w, out, b_mn_major=True, aux=aux, act=act)
    _status_ok()
    dh = dy.float() @ w.float()
    x = aux.float().requires_grad_(True)
    f = {"relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu}[name]
    f(x).sum().backward()
    assert _rel_err(out, dh * x.grad) < 1.5e-2


@pytest.mark.parametrize("split_k", [0, 1, 4])
def test_gemm_wgrad_fp32_accumulate_split_k(split_k):
    torch.manual_seed(6)
    tokens, n_out, k_in = 4000, 1024, 1024
    dy = torch.randn(tokens, n_out, device=DEV).bfloat16()
    x = torch.randn(tokens, k_in, device=DEV).bfloat16()
    acc = torch.ones(n_out, k_in, device=DEV)
    ops.gemm(dy, x, acc, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True, split_k=split_k)
    _status_ok()
    want = dy.float().t() @ x.float() + 1.0
    assert _rel_err(acc, want) < 5e-3


@pytest.mark.parametrize("tokens,n_out,k_in", [(8192, 3072, 1024), (8000, 4096, 1024), (5000, 1280, 768), (8192, 1024, 2048)])
@pytest.mark.parametrize("stream_k", [1, 0])
def test_gemm_wgrad_equal_runs_of_k_blocks(tokens, n_out, k_in, stream_k):
    """Weight gradients whose tiles do not fill the CTA pairs evenly are split into equal runs of k-blocks that may
    end inside a tile; the partial tiles meet in the fp32 output through reductions.  Same result either way."""
    torch.manual_seed(7)
    dy = torch.randn(tokens, n_out, device=DEV).bfloat16()
    x = torch.randn(tokens, k_in, device=DEV).bfloat16()
    acc = torch.full((n_out, k_in), 0.5, device=DEV)
    ops.ext().set_gemm_variant(40 + stream_k)
    try:
        ops.gemm(dy, x, acc, a_mn_major=True, b_mn_major=True, accumulate=True, allow_split_k=True)
    finally:
        ops.ext().set_gemm_variant(41)
    _status_ok()
    want = dy.float().t() @ x.float() + 0.5
    assert _rel_err(acc, want) < 5e-3


@pytest.mark.parametrize("M,N,K", [(256, 1024, 1024), (256, 1000, 512), (64, 4096, 1024), (256, 32000, 1024)])
def test_gemm_decode_shapes_bias_and_transposed_weight(M, N, K):
    """Few-row problems take 64-column tiles (many CTAs stream the weight matrix); bias epilogue, ragged N."""
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, w, out, bias=bias, act=1)
    torch.cuda.synchronize()
    _status_ok()
    want = torch.relu(a.float() @ w.float().t() + bias.float())
    assert _rel_err(out, want) < 1e-2
    wt = w.t().contiguous()                      # [K, N]: the same weights stored N-contiguous
    if N % 8 == 0:
        out2 = torch.empty_like(out)
        ops.gemm(a, wt, out2, b_mn_major=True, bias=bias, act=1)
        torch.cuda.synchronize()
        _status_ok()
        assert _rel_err(out2, want) < 1e-2


def test_gemm_sign_bit_mask_round_trip():
    """Forward epilogue writes one sign bit per output; the mask-backward epilogue applies it to another product."""
    torch.manual_seed(0)
    M, N, K = 300, 1000, 256
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    bits = torch.zeros(M, (N + 31) // 32, dtype=torch.int32, device=DEV)
    ops.gemm(a, w, out, act=1, mask=bits)
    torch.cuda.synchronize()
    positive = out.float() > 0
    cols = torch.arange(N, device=DEV)
    got = ((bits[:, cols // 32] >> (cols % 32)) & 1).bool()
    assert torch.equal(got, positive)
    g = torch.randn(M, 64, device=DEV).bfloat16()
    w2 = torch.randn(N, 64, device=DEV).bfloat16()
    d = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(g, w2, d, act=8, mask=bits, alpha=1.25)
    torch.cuda.synchronize()
    _status_ok()
    want = (g.float() @ w2.float().t()) * 1.25 * positive
    assert _rel_err(d, want) < 1e-2


@pytest.mark.parametrize("M,N,K", [(8192, 4096, 1024), (1000, 1024, 512), (300, 264, 256), (129, 64, 128)])
def test_gemm_column_sums_in_the_epilogue(M, N, K):
    """The sign-bit backward epilogue also adds the column sums of its bf16 output to an fp32 vector (bias gradient)."""
    torch.manual_seed(9)
    dy = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(K, N, device=DEV) * 0.05).bfloat16()            # [K, N]: B read MN-major, as in the fc2 data gradient
    bits = torch.randint(-2 ** 31, 2 ** 31 - 1, (M, (N + 31) // 32), device=DEV, dtype=torch.int32)
    out = ops.empty_rows(M, N, DEV)
    gb = torch.full((N,), 0.25, device=DEV)
    ops.gemm(dy, w, out, b_mn_major=True, act=8, mask=bits, alpha=1.1, colsum=gb)
    _status_ok()
    ref = torch.empty_like(out)
    ops.gemm(dy, w, ref, b_mn_major=True, act=8, mask=bits, alpha=1.1)
    assert torch.equal(out, ref)
    want = ref.float().sum(0) + 0.25
    assert (gb - want).abs().max().item() <= 2e-3 * max(1.0, want.abs().max().item())


def test_sm_reserve_only_changes_the_grid():
    """SMs set aside for communication kernels: every launcher sizes its grid for the rest; results do not change."""
    torch.manual_seed(9)
    a = torch.randn(2048, 512, device=DEV).bfloat16()
    b = torch.randn(1024, 512, device=DEV).bfloat16()
    want = torch.empty(2048, 1024, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, want)
    try:
        ops.ext().set_sm_reserve(8)
        got = torch.empty_like(want)
        ops.gemm(a, b, got)
        x = torch.randn(4096, 1024, device=DEV).bfloat16()
        g = torch.ones(1024, device=DEV).bfloat16()
        y = ops.ext().layernorm_fwd(x, g, torch.zeros_like(g), 1e-5)[0] if hasattr(ops.ext(), "layernorm_fwd") else None
    finally:
        ops.ext().set_sm_reserve(0)
    _status_ok()
    assert torch.equal(got, want)
    if y is not None:
        assert torch.isfinite(y.float()).all()

"""The matrix product that gathers its own weight operand (fully sharded parameters), on one GPU.

With a world of one the "owners" of all pieces are this GPU, so the whole in-kernel path runs - the epilogue warps
copying 4 KB blocks from the shard into the staging buffer, the segment counters, the TMA producer waiting on them,
the counters' reset - without a second device.  Several emulated ranks are one kernel over all ranks' shards here
(separate shard buffers on the same GPU), which is the layout the multi-GPU tests use with peer pointers.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sharded_case(n_out, n_in, world, unit_off=128, seed=0):
    torch.manual_seed(seed)
    dev = "cuda"
    w = (torch.randn(n_out, n_in, device=dev) * 0.05).bfloat16()
    unit_len = unit_off + w.numel() + 192
    piece = (-(-unit_len // world) + 63) // 64 * 64
    unit = torch.zeros(piece * world, device=dev, dtype=torch.bfloat16)
    unit[unit_off:unit_off + w.numel()] = w.reshape(-1)
    shard_off = 256
    shards = [torch.full((shard_off + piece,), 7.0, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    for r in range(world):
        shards[r][shard_off:shard_off + piece] = unit[r * piece:(r + 1) * piece]
    staging = torch.full((piece * world,), float("nan"), device=dev, dtype=torch.bfloat16)
    counters = torch.zeros(4096 + 8, dtype=torch.int32, device=dev)
    view = staging[unit_off:unit_off + w.numel()].view(n_out, n_in)
    gather = (0, [s.data_ptr() for s in shards], staging, shard_off, piece, unit_off, w.numel(), counters)
    return w, view, gather, counters, shards


class _Rec:
    def __init__(self, g):
        self.g = g

    def pending(self):
        return self.g


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("m,n_out,n_in", [(1024, 768, 512), (8192, 3072, 1024), (300, 256, 1280), (96, 512, 512)])
def test_forward_product_gathers_its_weight(world, m, n_out, n_in):
    from nmtgminor_b200 import ops
    w, view, gather, counters, _keep = _sharded_case(n_out, n_in, world)
    x = torch.randn(m, n_in, device="cuda").bfloat16()
    want = torch.empty(m, n_out, device="cuda", dtype=torch.bfloat16)
    ops.gemm(x, w, want)
    got = torch.empty_like(want)
    for _ in range(2):          # twice: the kernel must leave its counters ready for the next launch
        view.fill_(float("nan"))
        ops.gemm(x, view, got, gather=_Rec(gather))
        torch.cuda.synchronize()
        assert ops.check_status() == 0
        assert torch.equal(view, w), "the staging copy differs from the sharded matrix"
        assert torch.equal(got, want)
        assert int(counters.abs().sum()) == 0
    ref = (x.float() @ w.float().t())
    assert (got.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("m,n_out,n_in", [(2048, 1024, 4096), (8192, 4096, 1024), (640, 1280, 256)])
def test_data_gradient_product_gathers_its_weight(world, m, n_out, n_in):
    """dx = dy W with W[n_out, n_in] as the MN-major operand: segments are 64-row bands of W."""
    from nmtgminor_b200 import ops
    w, view, gather, counters, _keep = _sharded_case(n_out, n_in, world, seed=1)
    dy = torch.randn(m, n_out, device="cuda").bfloat16()
    want = torch.empty(m, n_in, device="cuda", dtype=torch.bfloat16)
    ops.gemm(dy, w, want, b_mn_major=True)
    got = torch.empty_like(want)
    view.fill_(float("nan"))
    ops.gemm(dy, view, got, b_mn_major=True, gather=_Rec(gather))
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    assert torch.equal(view, w)
    assert torch.equal(got, want)
    assert int(counters.abs().sum()) == 0
    ref = dy.float() @ w.float()
    assert (got.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-2


def test_unfused_switch_gives_the_same_result():
    from nmtgminor_b200 import ops
    w, view, gather, counters, _keep = _sharded_case(1024, 1024, 2, seed=2)
    x = torch.randn(512, 1024, device="cuda").bfloat16()
    a, b = torch.empty(512, 1024, device="cuda", dtype=torch.bfloat16), torch.empty(512, 1024, device="cuda", dtype=torch.bfloat16)
    ops.gemm(x, view, a, gather=_Rec(gather))
    ops.ext().set_gemm_variant(50)          # copy launch first, then the plain product
    try:
        view.fill_(float("nan"))
        ops.gemm(x, view, b, gather=_Rec(gather))
    finally:
        ops.ext().set_gemm_variant(51)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(view, w)

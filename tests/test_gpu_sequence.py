"""sm_100a sequence kernels against their fp32 PyTorch restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from nmtgminor_b200 import ops
from nmtgminor_b200.ops import sequence as S


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pack", [False, True])
@pytest.mark.parametrize("relu", [False, True])
def test_transducer_joint_fwd_bwd(dtype, pack, relu):
    torch.manual_seed(0)
    dev = _dev()
    B, T, U, H = 3, 9, 5, 64
    f = torch.randn(B, T, H, device=dev, dtype=dtype, requires_grad=True)
    g = torch.randn(B, U, H, device=dev, dtype=dtype, requires_grad=True)
    fl = torch.tensor([9, 4, 7], device=dev, dtype=torch.int32)
    gl = torch.tensor([5, 3, 1], device=dev, dtype=torch.int32)
    joint = S.TransducerJoint(pack_output=pack, relu=relu)
    out = joint(f, g, fl, gl)
    fr, gr = f.detach().float().requires_grad_(), g.detach().float().requires_grad_()
    ref = S.transducer_joint_reference(fr, gr, fl, gl, relu=relu, pack_output=pack)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert out.shape == ref.shape
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    # bf16 sums over up to 9 terms
    assert torch.allclose(f.grad.float(), fr.grad, atol=tol * 8, rtol=tol)
    assert torch.allclose(g.grad.float(), gr.grad, atol=tol * 8, rtol=tol)


def test_transducer_joint_dropout_consistent_mask():
    dev = _dev()
    B, T, U, H = 2, 6, 4, 128
    f = torch.randn(B, T, H, device=dev, requires_grad=True)
    g = torch.randn(B, U, H, device=dev, requires_grad=True)
    fl = torch.tensor([6, 5], device=dev, dtype=torch.int32)
    gl = torch.tensor([4, 2], device=dev, dtype=torch.int32)
    joint = S.TransducerJoint(relu=True, dropout=True, dropout_prob=0.25).train()
    out = joint(f, g, fl, gl)
    plain = S.transducer_joint_reference(f.detach(), g.detach(), fl, gl, relu=True)
    kept = out != 0
    frac = kept.float().sum() / (plain != 0).float().sum()
    assert 0.65 < frac.item() < 0.85
    scale = 256.0 / (256 - 64)
    assert torch.allclose(out[kept], plain[kept] * scale, rtol=1e-5, atol=1e-6)
    out.sum().backward()
    # gradient of f[b, t] = scale * number of kept positive entries over u
    expect = (kept.float() * scale).sum(2)
    assert torch.allclose(f.grad, expect, atol=1e-4)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("fuse", [False, True])
def test_transducer_loss(packed, fuse):
    torch.manual_seed(1)
    dev = _dev()
    B, T, U, V = 3, 7, 5, 11
    fl = torch.tensor([7, 5, 6], device=dev, dtype=torch.int32)
    yl = torch.tensor([4, 2, 3], device=dev, dtype=torch.int32)
    label = torch.randint(1, V, (B, U - 1), device=dev, dtype=torch.int32)
    logits = torch.randn(B, T, U, V, device=dev)
    zr = logits.clone().requires_grad_()
    ref = S.transducer_loss_reference(torch.log_softmax(zr, -1), label.long(), fl, yl, 0)
    ref.sum().backward()
    z = logits.clone().requires_grad_()
    loss_mod = S.TransducerLoss(fuse_softmax_backward=fuse, packed_input=packed)
    if packed:
        rows = [z[b, :int(fl[b]), :int(yl[b]) + 1].reshape(-1, V) for b in range(B)]
        zin = torch.cat(rows, 0)
    else:
        zin = z
    if fuse:
        loss = loss_mod.forward_logits(zin, label, fl, yl, 0, max_f_len=T)
    else:
        loss = loss_mod(torch.log_softmax(zin, -1), label, fl, yl, 0, max_f_len=T)
    assert torch.allclose(loss, ref.detach(), atol=1e-4, rtol=1e-5)
    loss.sum().backward()
    assert torch.allclose(z.grad, zr.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("direction", [0, 1, 2])
def test_lru_scan(direction):
    torch.manual_seed(2)
    dev = _dev()
    B, N, L = 3, 8, 100
    lam = torch.polar(torch.rand(N) * 0.5 + 0.45, torch.rand(N) * 6).to(dev).requires_grad_()
    x = torch.randn(B, N, L, dtype=torch.complex64, device=dev, requires_grad=True)
    lengths = torch.tensor([100, 33, 64], device=dev, dtype=torch.int32)
    h = S.lru_scan(lam, x, lengths, direction)
    lr, xr = lam.detach().cpu().requires_grad_(), x.detach().cpu().requires_grad_()
    ref = S.lru_scan_reference(lr, xr, lengths.cpu(), direction)
    assert torch.allclose(h.cpu(), ref, atol=1e-4, rtol=1e-4)
    w = torch.randn(B, N, L, dtype=torch.complex64)
    (h * w.to(dev)).real.sum().backward()
    (ref * w).real.sum().backward()
    assert torch.allclose(x.grad.cpu(), xr.grad, atol=1e-3, rtol=1e-3)
    assert torch.allclose(lam.grad.cpu(), lr.grad, atol=2e-2, rtol=1e-3)


def test_cauchy_fwd_bwd():
    torch.manual_seed(3)
    dev = _dev()
    I, Q, L, H, N = 2, 3, 40, 8, 16
    a = torch.randn(I, Q, H, N, dtype=torch.complex64, device=dev, requires_grad=True)
    b = (torch.randn(Q, L, H, dtype=torch.complex64, device=dev) + 4.0).requires_grad_()
    c = torch.randn(Q, N, dtype=torch.complex64, device=dev, requires_grad=True)
    out = S.cauchy_kernel_coefficient(a, b, c)
    ar, br, cr = (t.detach().clone().requires_grad_() for t in (a, b, c))
    ref = S.cauchy_reference(ar, br, cr)
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-4)
    w = torch.randn_like(ref)
    (out * w).real.sum().backward()
    (ref * w).real.sum().backward()
    for got, want in ((a.grad, ar.grad), (b.grad, br.grad), (c.grad, cr.grad)):
        assert torch.allclose(got, want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_mask_dropout(dtype):
    torch.manual_seed(4)
    dev = _dev()
    Bsz, heads, Tq, Tk = 2, 4, 5, 77
    x = torch.randn(Bsz * heads * Tq, Tk, device=dev, dtype=dtype, requires_grad=True)
    mask = torch.zeros(Bsz, Tk, dtype=torch.bool, device=dev)
    mask[1, 50:] = True
    yd, y = S.softmax_dropout(x, mask, rows_per_mask=heads * Tq, scale=0.5, p=0.0)
    xr = x.detach().float().requires_grad_()
    _, yr = S.softmax_dropout_reference(xr, mask, heads * Tq, 0.5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(y.float(), yr, atol=tol)
    w = torch.randn_like(yr)
    (yd.float() * w).sum().backward()
    (yr * w).sum().backward()
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol)
    # dropout: kept entries scaled, dropped entries zero, same mask in backward
    x2 = torch.randn(64, 256, device=dev, requires_grad=True)
    yd2, y2 = S.softmax_dropout(x2, None, 1, 1.0, p=0.5)
    kept = yd2 != 0
    assert 0.4 < kept.float().mean().item() < 0.6
    assert torch.allclose(yd2[kept], y2[kept] * 2.0, rtol=1e-5)
    yd2.sum().backward()
    g = kept.float() * 2.0
    expect = y2 * (g - (g * y2).sum(-1, keepdim=True))
    assert torch.allclose(x2.grad, expect, atol=1e-5)


def test_softmax_family_variants_on_the_kernels():
    """Time mask, additive mask, presampled dropout and the recompute backward against the fp32 PyTorch formulas."""
    torch.manual_seed(6)
    dev = _dev()
    B, H, Tq, Tk = 2, 3, 5, 90
    x = torch.randn(B, H, Tq, Tk, device=dev, requires_grad=True)
    lengths = torch.tensor([90, 41], device=dev)
    w = torch.randn(B, H, Tq, Tk, device=dev)

    def plain(xx, add=None, drop=None):
        s = xx * 0.5
        if add is not None:
            s = s + add
        s = s.masked_fill((torch.arange(Tk, device=dev)[None, :] >= lengths[:, None])[:, None, None, :], float("-inf"))
        y = torch.softmax(s, -1)
        return y * drop if drop is not None else y

    add = torch.randn(B, 1, 1, Tk, device=dev)
    drop = (torch.rand(B, H, Tq, Tk, device=dev) > 0.3).float() / 0.7
    for recompute in (False, True):
        xr = x.detach().clone().requires_grad_()
        got = S.masked_softmax_dropout(x, lengths=lengths, rows_per_mask=H * Tq, scale=0.5, additive_mask=add, drop_mask=drop,
                                       recompute=recompute)
        want = plain(xr, add, drop)
        assert torch.allclose(got, want, atol=1e-5), recompute
        x.grad = None
        (got * w).sum().backward()
        (want * w).sum().backward()
        assert torch.allclose(x.grad, xr.grad, atol=1e-5), recompute
    # kernel-drawn dropout with the recompute backward: the mask of the forward pass is regenerated
    x2 = torch.randn(32, 128, device=dev, requires_grad=True)
    yd = S.masked_softmax_dropout(x2, p=0.5, recompute=True)
    kept = yd != 0
    y = torch.softmax(x2.detach(), -1)
    assert torch.allclose(yd[kept], y[kept] * 2.0, rtol=1e-4)
    yd.sum().backward()
    g = kept.float() * 2.0
    assert torch.allclose(x2.grad, y * (g - (g * y).sum(-1, keepdim=True)), atol=1e-5)

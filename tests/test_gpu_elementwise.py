"""Memory-bound kernels against fp32 PyTorch restatements: LayerNorm, cross-entropy, dropout-add,
embedding, column sums, flat AdamW."""
import math

import pytest
import torch

from nmtgminor_b200 import ops
from nmtgminor_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, what):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), "%s: max abs err %g (ref max %g)" % (what, err, b.abs().max().item())


@pytest.mark.parametrize("rows,hidden", [(7, 256), (300, 512), (1000, 1024), (513, 1280), (64, 2048), (33, 264),
                                         (40, 4096), (700, 5120), (9, 2056), (5, 16384)])
def test_layernorm_fwd_bwd(rows, hidden):
    torch.manual_seed(0)
    x = (torch.randn(rows, hidden, device=DEV) * 2 + 0.5).bfloat16()
    g = (torch.randn(hidden, device=DEV) * 0.2 + 1).bfloat16()
    b = (torch.randn(hidden, device=DEV) * 0.2).bfloat16()
    dy = torch.randn(rows, hidden, device=DEV).bfloat16()
    dres = torch.randn(rows, hidden, device=DEV).bfloat16()
    y, mean, rstd = ops.ext().layernorm_fwd(x, g, b, 1e-5)
    xf = x.float().requires_grad_(True)
    gf, bf = g.float().requires_grad_(True), b.float().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xf, (hidden,), gf, bf, 1e-5)
    _close(y, yr, 3e-2, 2e-2, "ln fwd")
    _close(mean, xf.mean(-1), 1e-3, 1e-3, "ln mean")
    yr.backward(dy.float())
    dgamma = torch.zeros(hidden, device=DEV)
    dbeta = torch.zeros(hidden, device=DEV)
    dx = ops.ext().layernorm_bwd(dy, x, mean, rstd, g, dres, dgamma, dbeta)
    _close(dx, xf.grad + dres.float(), 6e-2, 3e-2, "ln dx")
    _close(dgamma, gf.grad, 0.02 * math.sqrt(rows) + 0.05, 2e-2, "ln dgamma")
    _close(dbeta, bf.grad, 0.02 * math.sqrt(rows) + 0.05, 2e-2, "ln dbeta")


@pytest.mark.parametrize("rows,vocab", [(64, 8000), (129, 32000), (16, 51865 + 7), (8, 250056)])
@pytest.mark.parametrize("smoothing", [0.0, 0.1])
def test_xent_fused(rows, vocab, smoothing):
    torch.manual_seed(1)
    vocab = vocab // 8 * 8
    logits = (torch.randn(rows, vocab, device=DEV) * 3).bfloat16()
    labels = torch.randint(1, vocab, (rows,), device=DEV)
    labels[::5] = 0  # padding rows
    lf = logits.float().requires_grad_(True)
    loss_r, correct_r, row_r = ref.cross_entropy(lf, labels, smoothing, 0)
    loss_r.sum().backward()
    work = logits.clone()
    loss_sum = torch.zeros(1, device=DEV)
    correct = torch.zeros(1, device=DEV)
    row = ops.ext().xent_fused(work, labels, smoothing, 0, loss_sum, correct, None, 1.0, True)
    _close(row, row_r, 2e-2, 1e-3, "xent row loss")
    _close(loss_sum, loss_r, 2e-2 * rows, 1e-3, "xent loss sum")
    assert correct.item() == correct_r.item()
    _close(work, lf.grad, 4e-3, 2e-2, "xent grad")
    assert work[::5].abs().max().item() == 0.0


def test_xent_grad_scale_tensor():
    torch.manual_seed(2)
    logits = torch.randn(32, 4096, device=DEV).bfloat16()
    labels = torch.randint(1, 4096, (32,), device=DEV)
    a, b = logits.clone(), logits.clone()
    ops.ext().xent_fused(a, labels, 0.1, 0, None, None, None, 1.0, True)
    gs = torch.full((1,), 0.25, device=DEV)
    ops.ext().xent_fused(b, labels, 0.1, 0, None, None, gs, 2.0, True)
    _close(b, a.float() * 0.5, 2e-3, 2e-2, "xent scaled grad")


@pytest.mark.parametrize("p", [0.1, 0.3])
def test_dropout_add_statistics_and_replay(p):
    torch.manual_seed(3)
    n = 1 << 20
    x = torch.ones(n, device=DEV).bfloat16()
    res = torch.full((n,), 2.0, device=DEV).bfloat16()
    y1 = ops.ext().dropout_add(x, res, p, 11, 5)
    y2 = ops.ext().dropout_add(x, res, p, 11, 5)
    assert torch.equal(y1, y2), "same (seed, stream) must reproduce the mask"
    y3 = ops.ext().dropout_add(x, res, p, 11, 6)
    assert not torch.equal(y1, y3)
    kept = (y1.float() - 2.0) > 0
    thr = int(p * 256 + 0.5)
    assert abs(kept.float().mean().item() - (256 - thr) / 256) < 5e-3
    scale = 256.0 / (256 - thr)
    _close((y1.float() - 2.0)[kept], torch.full_like(y1.float()[kept], scale), 2e-2, 0, "keep scale")
    # backward = same mask on the gradient
    dy = torch.randn(n, device=DEV).bfloat16()
    dx = ops.ext().dropout_add(dy, None, p, 11, 5)
    _close(dx, dy.float() * kept * scale, 2e-2, 1e-2, "dropout backward")


def test_embedding_fwd_bwd():
    torch.manual_seed(4)
    V, H, N = 1000, 256, 700
    table = torch.randn(V, H, device=DEV).bfloat16()
    pos_table = torch.randn(128, H, device=DEV).bfloat16()
    tokens = torch.randint(0, V, (N,), device=DEV)
    positions = torch.randint(0, 128, (N,), device=DEV)
    out = ops.ext().embed_fwd(tokens, positions, table, pos_table, 16.0, 0.0, 1, 1)
    want = table.float()[tokens] * 16.0 + pos_table.float()[positions]
    _close(out, want, 0.3, 1e-2, "embed fwd")
    dy = torch.randn(N, H, device=DEV).bfloat16()
    dtab = torch.zeros(V, H, device=DEV)
    dpos = torch.zeros(128, H, device=DEV)
    ops.ext().embed_bwd(tokens, positions, dy, dtab, dpos, 16.0, 0.0, 1, 1, 0)
    want_t = torch.zeros(V, H, device=DEV).index_add_(0, tokens, dy.float() * 16.0 * (tokens != 0)[:, None])
    want_p = torch.zeros(128, H, device=DEV).index_add_(0, positions, dy.float() * (tokens != 0)[:, None])
    _close(dtab, want_t, 1e-2, 1e-3, "embed dtable")
    _close(dpos, want_p, 1e-2, 1e-3, "embed dpos")


def test_colsum():
    torch.manual_seed(5)
    x = torch.randn(3000, 1026, device=DEV).bfloat16()
    out = torch.ones(1026, device=DEV)
    ops.ext().colsum(x, out)
    _close(out, x.float().sum(0) + 1, 5e-2, 1e-3, "colsum")


@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 256), (1000, 1024), (8148, 1024), (513, 4096), (300, 512)])
def test_dropout_colsum_matches_two_passes(rows, cols):
    torch.manual_seed(2)
    x = torch.randn(rows, cols, device=DEV).bfloat16()
    want_y = ops.ext().dropout_add(x, None, 0.3, 99, 5)
    want_sum = torch.full((cols,), 2.0, device=DEV)
    ops.ext().colsum(want_y, want_sum)
    got_sum = torch.full((cols,), 2.0, device=DEV)
    got_y = ops.ext().dropout_colsum(x, 0.3, 99, 5, got_sum)
    assert torch.equal(got_y, want_y)
    _close(got_sum, want_y.float().sum(0) + 2, 1e-3 * math.sqrt(rows) + 1e-3, 1e-4, "dropout_colsum vs fp32")
    _close(got_sum, want_sum, 5e-2, 1e-3, "dropout_colsum vs colsum")


@pytest.mark.parametrize("decoupled,clip", [(True, 0.0), (False, 0.0), (True, 0.5)])
def test_adamw_flat(decoupled, clip):
    torch.manual_seed(6)
    n = 1 << 16
    master = torch.randn(n, device=DEV)
    grad = torch.randn(n, device=DEV) * 0.01
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    work = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    rm, rg, rmm, rv = master.clone(), grad.clone(), m.clone(), v.clone()
    wd = 0.01
    for step in (1, 2, 3):
        hyper = torch.zeros(16)
        hyper[0], hyper[1], hyper[2], hyper[3] = 1e-2, 0.9, 0.997, 1e-9
        hyper[4], hyper[5], hyper[6], hyper[7], hyper[8] = wd, 1 - 0.9 ** step, 1 - 0.997 ** step, 0.5, clip
        hi = hyper.view(torch.int32)
        hi[9], hi[10] = int(decoupled), 1
        hyper = hyper.to(DEV)
        sq = torch.zeros(1, device=DEV)
        bad = torch.zeros(1, device=DEV, dtype=torch.int32)
        ops.ext().sq_norm(grad, sq, bad)
        _close(sq, grad.pow(2).sum().reshape(1), 1e-3, 1e-4, "sq norm")
        ops.ext().adamw_flat(master, work, grad, m, v, hyper, sq, bad)
        ref.adamw_step(rm, rg, rmm, rv, lr=1e-2, beta1=0.9, beta2=0.997, eps=1e-9, weight_decay=wd, step=step,
                       grad_scale=0.5, max_grad_norm=clip, decoupled=decoupled)
        _close(master, rm, 1e-5, 1e-4, "adam master step %d" % step)
        _close(work, rm, 1e-2, 1e-2, "adam bf16 copy")
        assert grad.abs().max().item() == 0.0, "gradient buffer must be cleared"
        grad = torch.randn(n, device=DEV) * 0.01
        rg = grad.clone()


def test_adamw_skips_on_nonfinite():
    n = 4096
    master = torch.ones(n, device=DEV)
    grad = torch.ones(n, device=DEV)
    grad[7] = float("inf")
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    hyper = torch.zeros(16)
    hyper[0], hyper[1], hyper[2], hyper[3], hyper[5], hyper[6], hyper[7] = 1e-2, 0.9, 0.997, 1e-9, 0.1, 0.003, 1.0
    hyper.view(torch.int32)[10] = 1
    sq = torch.zeros(1, device=DEV)
    bad = torch.zeros(1, device=DEV, dtype=torch.int32)
    ops.ext().sq_norm(grad, sq, bad)
    assert bad.item() == 1
    ops.ext().adamw_flat(master, None, grad, m, v, hyper.to(DEV), sq, bad)
    assert torch.equal(master, torch.ones(n, device=DEV)) and grad.abs().max().item() == 0.0


def test_layernorm_residual_pair_sums_both_gradient_paths():
    """``(x, LN(x))`` as one autograd node: d/dx of ``a * x + b * LN(x)`` matches the fp32 composition."""
    from nmtgminor_b200.models.layers import LayerNorm
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    torch.manual_seed(3)
    ln = LayerNorm(512)
    with torch.no_grad():
        ln.weight.normal_(1.0, 0.2)
        ln.bias.normal_(0.0, 0.2)
    store = FlatParameterStore(ln, DEV)
    x = torch.randn(300, 512, device=DEV).bfloat16().requires_grad_(True)
    wa, wb = torch.randn(300, 512, device=DEV).bfloat16(), torch.randn(300, 512, device=DEV).bfloat16()
    res, h = ln.with_residual(x)
    assert type(h.grad_fn).__name__.startswith("_LayerNormResidualFn")
    (res * wa + h * wb).sum().backward()
    xf = x.detach().float().requires_grad_(True)
    gf, bf = ln.weight.detach().float().requires_grad_(True), ln.bias.detach().float().requires_grad_(True)
    hf = torch.nn.functional.layer_norm(xf, (512,), gf, bf, 1e-5)
    (xf * wa.float() + hf * wb.float()).sum().backward()
    _close(x.grad, xf.grad, 8e-2, 3e-2, "ln residual dx")
    _close(ln.weight.main_grad, gf.grad, 0.02 * math.sqrt(300) + 0.05, 2e-2, "ln residual dgamma")
    # only the residual path used: the gradient passes straight through
    x2 = x.detach().clone().requires_grad_(True)
    res2, _ = ln.with_residual(x2)
    (res2 * wa).sum().backward()
    assert torch.equal(x2.grad, wa)
    del store


@pytest.mark.parametrize("act", [1, 2, 3], ids=["relu", "gelu", "silu"])
@pytest.mark.parametrize("p", [0.0, 0.2])
def test_act_backward_one_pass(act, p):
    """dz = dropout-mask(dy) * act'(z) against the two-step PyTorch statement, and through ``ops.linear`` with autograd."""
    from nmtgminor_b200.ops import _act_backward
    torch.manual_seed(5)
    rows, cols = 304, 264
    dy = torch.randn(rows, cols, device=DEV).bfloat16()
    z = (torch.randn(rows, cols, device=DEV) * 2).bfloat16()
    got = ops.ext().act_backward(dy, z, act, p, 17, 4)
    masked = ops.ext().dropout_add(dy, None, p, 17, 4) if p > 0 else dy
    want = _act_backward(masked, z, act)
    _close(got, want, 2e-2, 2e-2, "act backward")
    assert ops.check_status() == 0
    # a linear layer with an activation trained through autograd agrees with the fp32 statement
    name = {1: "relu", 2: "gelu", 3: "silu"}[act]
    lin = torch.nn.Linear(cols, 128).to(DEV)
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    FlatParameterStore(lin, torch.device(DEV))
    x = torch.randn(rows, cols, device=DEV).bfloat16().requires_grad_(True)
    y = ops.linear(x, lin.weight, lin.bias, name, 0.0, None, True)
    y.float().square().sum().backward()
    xr = x.detach().float().requires_grad_(True)
    w, b = lin.weight.work.float(), lin.bias.work.float()
    zr = xr @ w.t() + b
    yr = {1: torch.relu, 2: torch.nn.functional.gelu, 3: torch.nn.functional.silu}[act](zr)
    yr.square().sum().backward()
    _close(x.grad, xr.grad, 0.15 * xr.grad.abs().max().item(), 5e-2, "linear+act input gradient")

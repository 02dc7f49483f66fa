"""CPU checks of the PyTorch restatements of the sequence ops (the oracles of the GPU tests)."""
import itertools
import math

import torch

from nmtgminor_b200.ops import sequence as S


def _brute_rnnt(x, label, T, U, blank):
    # enumerate all monotone paths: T blanks and U-1 labels, the last symbol is the final blank
    total = []
    for labs_at in itertools.combinations(range(T + U - 2), U - 1):
        t = u = 0
        lp = 0.0
        for s in range(T + U - 2):
            if s in labs_at:
                lp += x[t, u, label[u]].item(); u += 1
            else:
                lp += x[t, u, blank].item(); t += 1
        lp += x[T - 1, U - 1, blank].item()
        total.append(lp)
    return -torch.logsumexp(torch.tensor(total), 0)


def test_transducer_loss_reference_matches_path_enumeration():
    torch.manual_seed(0)
    T, U, V = 4, 3, 5
    x = torch.log_softmax(torch.randn(1, T, U, V), -1)
    label = torch.tensor([[1, 3]])
    loss = S.transducer_loss_reference(x, label, torch.tensor([T]), torch.tensor([U - 1]), 0)
    assert abs(loss.item() - _brute_rnnt(x[0], label[0], T, U, 0).item()) < 1e-5


def test_joint_reference_packing():
    f, g = torch.randn(2, 3, 4), torch.randn(2, 2, 4)
    fl, gl = torch.tensor([3, 2]), torch.tensor([2, 1])
    dense = S.transducer_joint_reference(f, g, fl, gl)
    packed = S.transducer_joint_reference(f, g, fl, gl, pack_output=True)
    assert packed.shape[0] == 3 * 2 + 2 * 1
    assert torch.equal(packed[:6].view(3, 2, 4), dense[0]) and torch.equal(packed[6:].view(2, 1, 4), dense[1, :2, :1])
    assert dense[1, 2].abs().sum() == 0
    assert S.batch_offsets(fl, gl).tolist() == [6, 8]


def test_lru_reference_and_module():
    torch.manual_seed(0)
    lam = torch.polar(torch.rand(4) * 0.9, torch.rand(4) * 3)
    x = torch.randn(2, 4, 6, dtype=torch.complex64)
    lengths = torch.tensor([6, 4])
    h = S.lru_scan(lam, x, lengths, 0)
    assert torch.allclose(h[0, :, 2], lam * (lam * x[0, :, 0] + x[0, :, 1]) + x[0, :, 2], atol=1e-5)
    hb = S.lru_scan(lam, x, lengths, 1)
    assert torch.allclose(hb[1, :, 2], lam * x[1, :, 3] + x[1, :, 2], atol=1e-5) and hb[1, :, 4:].abs().sum() == 0
    m = S.BLRU(8, 4)
    y = m(torch.randn(2, 6, 8), lengths)
    assert y.shape == (2, 6, 8)
    y.sum().backward()
    assert m.nu_log.grad is not None


def test_cauchy_and_softmax_reference():
    a = torch.randn(2, 3, 4, 5, dtype=torch.complex64)
    b = torch.randn(3, 6, 4, dtype=torch.complex64)
    c = torch.randn(3, 5, dtype=torch.complex64)
    out = S.cauchy_kernel_coefficient(a, b, c)
    assert out.shape == (2, 3, 6, 4)
    assert torch.allclose(out[1, 2, 3, 0], (a[1, 2, 0] / (b[2, 3, 0] - c[2])).sum(), atol=1e-4)
    k = S.compute_kernel_coefficient(torch.randn(6, 2), torch.randn(3, 5, dtype=torch.complex64), torch.rand(3, 4) + 0.5,
                                     torch.randn(3, 1, 4, 5), torch.randn(3, 2, 4, 5))
    assert k.shape == (3, 1, 2, 6, 4)
    x = torch.randn(2 * 3, 5)
    mask = torch.tensor([[0, 0, 0, 1, 1], [0, 0, 0, 0, 0]], dtype=torch.bool)
    yd, y = S.softmax_dropout(x, mask, rows_per_mask=3)
    assert torch.allclose(y.sum(-1), torch.ones(6)) and y[:3, 3:].abs().sum() == 0


def test_softmax_family_variants_on_the_reference_path():
    """Time mask, additive mask, presampled dropout and the recompute switch give the plain formulas (CPU statement)."""
    import torch
    from nmtgminor_b200.ops import sequence as S
    torch.manual_seed(0)
    x = torch.randn(2, 3, 5, 7)                               # [batch, heads, queries, keys]
    lengths = torch.tensor([7, 4])
    got = S.masked_softmax_dropout(x, lengths=lengths, rows_per_mask=15, scale=0.5)
    want = torch.softmax((x * 0.5).masked_fill((torch.arange(7)[None, :] >= lengths[:, None])[:, None, None, :], float("-inf")), -1)
    assert torch.allclose(got, want, atol=1e-6)
    add = torch.randn(2, 1, 1, 7)
    got = S.masked_softmax_dropout(x, additive_mask=add, scale=0.5)
    assert torch.allclose(got, torch.softmax(x * 0.5 + add, -1), atol=1e-6)
    drop = (torch.rand_like(x) > 0.3).float() / 0.7
    got = S.masked_softmax_dropout(x, drop_mask=drop)
    assert torch.allclose(got, torch.softmax(x, -1) * drop, atol=1e-6)
    assert torch.allclose(S.masked_softmax_dropout(x, recompute=True), torch.softmax(x, -1), atol=1e-6)
    assert S.time_mask_from_lengths(lengths, 7).tolist()[1] == [0, 0, 0, 0, 1, 1, 1]

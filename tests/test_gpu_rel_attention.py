"""Relative-position attention kernel against its fp32 PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from nmtgminor_b200 import ops
from nmtgminor_b200.ops.rel_attention import rel_self_attention, rel_self_attention_reference


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lens", [[5, 17, 1], [128, 64, 33, 100]])
def test_rel_attention_forward_backward(causal, lens):
    torch.manual_seed(0)
    dev = "cuda"
    heads, H = 2, 128
    N = sum(lens)
    cap = N + 5                                         # static padding rows at the end
    T = max(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    qkv = (0.5 * torch.randn(cap, 3 * H, device=dev)).bfloat16().requires_grad_()
    r = (0.5 * torch.randn(2 * T - 1, H, device=dev)).bfloat16().requires_grad_()
    u = (0.1 * torch.randn(heads, 64, device=dev)).requires_grad_()
    w = (0.1 * torch.randn(heads, 64, device=dev)).requires_grad_()
    out = rel_self_attention(qkv, r, u, w, cu, heads, T, T - 1, causal, 0.0)
    ref_in = [t.detach().float().requires_grad_() for t in (qkv, r, u, w)]
    ref = rel_self_attention_reference(ref_in[0], ref_in[1], ref_in[2], ref_in[3], cu, heads, T - 1, causal)
    assert (out.float()[:N] - ref[:N]).abs().max().item() < 2e-2
    assert out[N:].abs().sum().item() == 0
    g = torch.randn_like(ref)
    g[N:] = 0
    (out.float() * g).sum().backward()
    (ref * g).sum().backward()
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-6)).item()
    assert rel(qkv.grad, ref_in[0].grad) < 3e-2
    assert rel(r.grad, ref_in[1].grad) < 3e-2
    assert rel(u.grad, ref_in[2].grad) < 3e-2
    assert rel(w.grad, ref_in[3].grad) < 3e-2


def test_rel_attention_dropout_is_consistent():
    torch.manual_seed(1)
    dev = "cuda"
    heads, H, T = 2, 128, 40
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    qkv = torch.zeros(T, 3 * H, device=dev).bfloat16()
    qkv[:, 2 * H:] = 1.0                                # v = 1: ctx = sum of (dropped) probabilities
    qkv.requires_grad_()
    r = torch.zeros(2 * T - 1, H, device=dev).bfloat16()
    u = torch.zeros(heads, 64, device=dev)
    out = rel_self_attention(qkv, r, u, u.clone(), cu, heads, T, T - 1, False, 0.5)
    sums = out.float()[:, 0]
    # uniform attention, each probability kept with chance 1/2 and doubled: row sums spread around 1
    assert 0.8 < sums.mean().item() < 1.2 and sums.std().item() > 0.05
    out.float().sum().backward()
    assert torch.isfinite(qkv.grad.float()).all()

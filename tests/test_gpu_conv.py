"""Convolution-as-GEMM (overlapping-row TMA view) against F.conv1d."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from nmtgminor_b200 import ops
from nmtgminor_b200.ops import conv as C
from nmtgminor_b200.parallel.flat import FlatParameterStore


@pytest.mark.parametrize("Ci,Co,k,s,act", [(512, 512, 3, 2, "gelu"), (512, 512, 2, 2, "none"), (80, 256, 3, 1, "gelu"),
                                           (256, 256, 3, 2, "relu")])
def test_conv1d_gemm_forward_backward(Ci, Co, k, s, act):
    torch.manual_seed(0)
    B, T = 3, 101
    conv = torch.nn.Conv1d(Ci, Co, k, stride=s).cuda()
    ref = torch.nn.Conv1d(Ci, Co, k, stride=s).cuda()
    ref.load_state_dict(conv.state_dict())
    store = FlatParameterStore(conv, "cuda")
    x = torch.randn(B, T, Ci, device="cuda").bfloat16().requires_grad_()
    y = C.conv1d(x, conv.weight, conv.bias, s, act)
    xr = x.detach().float().requires_grad_()
    with torch.no_grad():
        ref.weight.copy_(conv.weight.work.float())
        ref.bias.copy_(conv.bias.work.float())
    yr = C.conv1d_reference(xr, ref.weight, ref.bias, s, act)
    assert y.shape == yr.shape
    scale = yr.abs().max().item()
    assert (y.float() - yr).abs().max().item() / scale < 2e-2
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    rel = lambda a, b: ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()
    assert rel(x.grad.float(), xr.grad) < 3e-2
    assert rel(conv.weight.main_grad, ref.weight.grad) < 3e-2
    assert rel(conv.bias.main_grad, ref.bias.grad) < 3e-2
    print("overlapping-row descriptors accepted:", C._OVERLAP_OK[0])


def test_feature_extractor_gemm_path_matches_library_path():
    from nmtgminor_b200.models.speech_encoders import ConvFeatureExtractor
    torch.manual_seed(0)
    specs = [(64, 10, 5), (64, 3, 2), (64, 3, 2), (64, 2, 2)]
    for mode in ("layer_norm", "default"):
        fe = ConvFeatureExtractor(specs, mode=mode, conv_bias=True).cuda()
        wav = torch.randn(2, 4000, device="cuda")
        want = fe(wav)                     # library path (no working copies yet)
        FlatParameterStore(fe, "cuda")
        got = fe(wav)
        assert got.shape == want.shape
        assert (got.float() - want).abs().max().item() / want.abs().max().item() < 5e-2

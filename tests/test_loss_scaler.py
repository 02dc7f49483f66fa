"""Dynamic loss scale: growth / back-off rule, checkpoint state, the CPU trainer path that skips an overflowing step, and
(GPU) the device-resident protocol around the fused optimiser."""
import math

import pytest
import torch

from nmtgminor_b200.options import default_options
from nmtgminor_b200.train.loss_scaler import DynamicLossScaler, wants_loss_scaling


def test_rule_and_state_dict():
    s = DynamicLossScaler("cpu", init_scale=1024.0, growth_interval=3)
    clean, bad = torch.zeros(1, dtype=torch.int32), torch.ones(1, dtype=torch.int32)
    for _ in range(2):
        s.update(nonfinite=clean)
    assert s.get_scale() == 1024.0
    s.update(nonfinite=clean)
    assert s.get_scale() == 2048.0
    s.update(nonfinite=bad)
    assert s.get_scale() == 1024.0 and s.skipped_steps() == 1
    s.update(norm=torch.tensor([-1.0]))
    assert s.get_scale() == 512.0 and s.skipped_steps() == 2
    s.update(norm=torch.tensor([3.0]))
    assert s.get_scale() == 512.0
    sd = s.state_dict()
    t = DynamicLossScaler("cpu")
    t.load_state_dict(sd)
    assert t.get_scale() == 512.0 and t.growth_interval == 3 and t.state_dict()["growth_tracker"] == 1
    assert float(t.state[2]) == 1.0 / 512.0
    assert float(s.scale) == 512.0 and s.scale.data_ptr() == s.state.data_ptr()
    # floor and ceiling
    lo = DynamicLossScaler("cpu", init_scale=1.0)
    lo.update(nonfinite=bad)
    assert lo.get_scale() == 1.0


def test_flag_selects_the_protocol():
    assert wants_loss_scaling(default_options(["-fp16"]))
    assert not wants_loss_scaling(default_options(["-fp16", "-bf16"]))
    assert not wants_loss_scaling(default_options([]))


def test_cpu_engine_skips_an_overflowing_step_and_halves_the_scale():
    from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.train.engine import TrainEngine
    torch.manual_seed(0)
    d = synthetic_dict(50)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-fp16", "-optim", "adam",
                           "-learning_rate", "0.01", "-update_method", "regular", "-dropout", "0", "-attn_dropout", "0",
                           "-word_dropout", "0", "-emb_dropout", "0"])
    model = build_model(opt, {"src": d, "tgt": d})
    eng = TrainEngine(model, opt, "cpu")
    assert eng.scaler is not None and eng.optim.loss_scaler is eng.scaler
    batches = token_budget_batches(50, 3, 8, 60, 3, seed=1)
    before = [p.detach().clone() for p in model.parameters()]
    eng.train_step(batches[0])
    assert eng.scaler.skipped_steps() == 0 and eng.optim._step == 1
    moved = [p.detach().clone() for p in model.parameters()]
    assert any(not torch.equal(a, b) for a, b in zip(before, moved))
    # the unscaled gradients are those of an unscaled run: compare one update with a scaler-free engine
    torch.manual_seed(0)
    opt2 = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-optim", "adam",
                            "-learning_rate", "0.01", "-update_method", "regular", "-dropout", "0", "-attn_dropout", "0",
                            "-word_dropout", "0", "-emb_dropout", "0"])
    model2 = build_model(opt2, {"src": d, "tgt": d})
    eng2 = TrainEngine(model2, opt2, "cpu")
    eng2.train_step(batches[0])
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.allclose(a, b, atol=2e-5), "loss scaling must not change the update"
    # overflow: a scale so large that the fp32 gradients become infinite
    eng.scaler.state[0] = 3.0e38
    eng.scaler.state[2] = 1.0 / 3.0e38
    eng.train_step(batches[1])
    assert eng.scaler.skipped_steps() == 1 and eng.optim._step == 1
    assert math.isclose(eng.scaler.get_scale(), 1.5e38, rel_tol=1e-6)
    for a, b in zip(model.parameters(), moved):
        assert torch.equal(a, b), "a skipped step leaves the parameters alone"


@pytest.mark.gpu
def test_device_protocol_around_the_fused_optimiser():
    """An inf written into the flat gradient buffer from the host skips exactly one update and halves the scale; clean
    steps grow it after the interval; the gradient factor seen by the kernel is base / scale."""
    from nmtgminor_b200 import ops
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    from nmtgminor_b200.train.optim import Optim
    dev = torch.device("cuda")
    lin = torch.nn.Linear(64, 64).to(dev)
    store = FlatParameterStore(lin, dev)
    opt = default_options(["-optim", "adam", "-learning_rate", "0.1", "-update_method", "regular", "-max_grad_norm", "0"])
    optim = Optim(opt)
    optim.set_parameters(lin.parameters(), store)
    sc = DynamicLossScaler(dev, init_scale=256.0, growth_interval=2)
    optim.loss_scaler = sc
    ref = store.master.clone()
    g = torch.randn_like(store.grad)
    store.grad.copy_(g * 256.0)                  # gradients as the scaled loss would have produced them
    optim.step(1.0)
    torch.cuda.synchronize()
    assert abs(float(optim.hyper[7]) - 1.0 / 256.0) < 1e-9
    # first Adam step moves every touched weight by lr * sign(g)
    moved = (store.master - ref)[: g.numel()]
    assert torch.allclose(moved[g != 0], -0.1 * torch.sign(g[g != 0]), atol=1e-3)
    after_first = store.master.clone()
    store.grad.copy_(g * 256.0)
    store.grad[5] = float("inf")
    optim.step(1.0)
    torch.cuda.synchronize()
    assert torch.equal(store.master, after_first), "the overflowing step must be skipped"
    assert sc.get_scale() == 128.0 and sc.skipped_steps() == 1
    for _ in range(2):
        store.grad.copy_(g * sc.get_scale())
        optim.step(1.0)
    torch.cuda.synchronize()
    assert sc.get_scale() == 256.0 and not torch.equal(store.master, after_first)
    assert ops.check_status() == 0

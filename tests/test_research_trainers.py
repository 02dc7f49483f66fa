"""Continual-learning trainers and their building blocks on CPU."""
import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_dataset, synthetic_dict
from nmtgminor_b200.options import default_options
from nmtgminor_b200.train import research as R
from nmtgminor_b200.train.trainer import Trainer


def test_reservoir_is_uniform_and_bounded():
    res = R.Reservoir(max_samples=50, seed=0)
    for i in range(2000):
        res.add_sample((i % 3, i))
    assert len(res) == 50 and res.num_observed == 2000
    kept = sorted(v[1] for v in res.data.values())
    # uniform over the stream: about a quarter of the kept items come from each quarter
    assert 5 <= sum(k < 500 for k in kept) <= 22 and 5 <= sum(k >= 1500 for k in kept) <= 22
    assert sum(res.get_stats().values()) == 50
    clone = R.Reservoir(50)
    clone.load_state_dict(res.state_dict())
    assert clone.data == res.data and len(res.sample(3)) == 3


def test_agem_and_gem_projections():
    g = torch.tensor([1.0, -2.0, 0.5])
    ref = torch.tensor([0.0, 1.0, 0.0])
    assert R.project_agem(g, ref)
    assert abs(float(torch.dot(g, ref))) < 1e-6 and torch.allclose(g, torch.tensor([1.0, 0.0, 0.5]))
    assert not R.project_agem(g, torch.tensor([1.0, 0.0, 0.0]))
    torch.manual_seed(0)
    M = torch.randn(3, 20)
    g = -M.sum(0) + 0.1 * torch.randn(20)
    out = R.project2cone2(g.clone(), M, margin=0.0, eps=1e-6, iters=5000)
    assert bool((M @ out > -1e-3).all())
    # among feasible points the projection is closer to g than the obvious feasible point 0
    assert float((out - g).norm()) < float(g.norm())


def test_ewc_penalty_gradient():
    ewc = R.EWC(4, "cpu", importance=2.0)
    ewc.accumulate(torch.tensor([1.0, 2.0, 0.0, 1.0]))
    ewc.accumulate(torch.tensor([1.0, 0.0, 0.0, 3.0]))
    theta0 = torch.zeros(4)
    ewc.finalize(theta0)
    assert torch.allclose(ewc.fisher, torch.tensor([1.0, 2.0, 0.0, 5.0]))
    theta = torch.tensor([1.0, 1.0, 1.0, -1.0], requires_grad=True)
    ewc.penalty(theta).backward()
    g = torch.zeros(4)
    ewc.add_penalty_grad(g, theta.detach())
    assert torch.allclose(g, theta.grad)


def _opt(extra=()):
    return default_options(["-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64", "-ffn_activation", "relu",
                            "-tie_weights", "-join_embedding", "-optim", "adam", "-learning_rate", "0.01", "-update_method",
                            "regular", "-dropout", "0.0", "-batch_size_words", "200", "-save_model", "/tmp/nmtg_research/model",
                            "-log_interval", "1000", "-reservoir_size", "8"] + list(extra))


def _data(seed):
    return synthetic_dataset(60, 5, 12, 40, batch_size_words=200, seed=seed)


def test_trainer_selection():
    assert R.select_trainer(_opt()) is Trainer
    assert R.select_trainer(_opt(["-ocl_training"])) is R.OCLTrainer
    assert R.select_trainer(_opt(["-ocl_training", "-meta_learning"])) is R.MetaOCLTrainer
    assert R.select_trainer(_opt(["-ocl_training", "-bayes_by_backprop"])) is R.BayesianOCLTrainer
    assert R.select_trainer(_opt(["-ocl_training", "-vat_training", "1"])) is R.VATTrainer
    assert R.select_trainer(_opt(["-offline_cl_training"])) is R.OfflineCLTrainer


def _run(cls, extra, datasets):
    torch.manual_seed(0)
    d = synthetic_dict(40)
    tr = cls(-1, {"src": d, "tgt": d}, _opt(extra), init_distributed=False)
    before = tr.engine.store.master.clone()
    loss, _ = tr.train_epoch(datasets, None, 1)
    assert loss == loss and loss > 0
    assert not torch.equal(before, tr.engine.store.master)
    return tr


def test_ocl_trainer_with_agem_replay():
    tr = _run(R.OCLTrainer, ["-ocl_training", "-agem_training"], [_data(1), _data(2)])
    assert 0 < len(tr.reservoir) <= 8 and tr.reservoir.num_observed > 8
    assert set(tr.reservoir.get_stats()) <= {0, 1}


def test_gem_meta_bayes_vat_offline_trainers_step():
    _run(R.GEMTrainer, ["-ocl_training", "-gem_training"], [_data(1), _data(2)])
    _run(R.MetaOCLTrainer, ["-ocl_training", "-meta_learning"], [_data(3)])
    _run(R.BayesianOCLTrainer, ["-ocl_training", "-bayes_by_backprop"], [_data(4)])
    _run(R.VATTrainer, ["-ocl_training", "-vat_training", "1"], [_data(5)])
    tr = _run(R.OfflineCLTrainer, ["-offline_cl_training", "-ewc_importance", "10.0"], [_data(6), _data(7)])
    assert tr.ewc.anchor is not None and float(tr.ewc.fisher.sum()) > 0


def test_dual_primal_learning_moves_the_memory_multipliers():
    """``-dpl_training``: replayed batches are weighted by per-slot multipliers, which rise while the memory loss is
    above ``-dpl_epsilon`` and are clamped at zero when it is far below."""
    tr = _run(R.OCLTrainer, ["-ocl_training", "-dpl_training", "-dpl_epsilon", "0.0", "-dpl_count", "2"], [_data(11)])
    lam = tr.reservoir.lambdas
    assert set(lam) == set(tr.reservoir.data) and all(v >= 0 for v in lam.values())
    assert any(v > 1.0 for v in lam.values())          # every loss is above a zero constraint
    assert tr.engine.loss_weight == 1.0                 # the weight is reset after the replay batches
    tr.dpl_epsilon = 1e6                               # constraint satisfied by a wide margin: multipliers fall to zero
    for _ in range(40):
        tr.update_lambdas()
    assert max(tr.reservoir.lambdas.values()) == 0.0
    sd = tr.reservoir.state_dict()
    fresh = R.Reservoir(8)
    fresh.load_state_dict(sd)
    assert fresh.lambdas == tr.reservoir.lambdas


def test_offline_trainer_example_budget_and_finalisation(tmp_path):
    """``-max_examples_seen`` becomes whole epochs; ``-finalize_only`` averages the round's checkpoints, fills the replay
    memory and writes ``*_final.pt``, from which the next round restores the memory."""
    torch.manual_seed(0)
    d = synthetic_dict(40)
    dicts = {"src": d, "tgt": d}
    save = str(tmp_path / "r1" / "model")
    data, valid = _data(3), _data(4)
    n_batches = len(data)
    common = ["-offline_cl_training", "-save_model", save, "-save_every", "100000"]
    tr = R.OfflineCLTrainer(-1, dicts, _opt(common + ["-max_examples_seen", str(2 * n_batches + 1)]), init_distributed=False)
    tr.run(None, data, valid)
    assert tr.opt.epochs == 2 and tr.optim._step == 2 * n_batches
    import glob
    files = sorted(glob.glob(save + "_ppl_*.pt"))
    assert len(files) == 2
    with pytest.raises(ValueError, match="finalize_only"):
        R.OfflineCLTrainer(-1, dicts, _opt(common + ["-max_examples_seen", "1"]), init_distributed=False).run(None, data, valid)
    fin = R.OfflineCLTrainer(-1, dicts, _opt(common + ["-finalize_only"]), init_distributed=False)
    name = fin.run(None, data, valid)
    assert name == save + "_final.pt" and fin.optim._step == 0
    ck = torch.load(name, weights_only=False)
    a, b = (torch.load(f, weights_only=False)["model"] for f in files)
    k = next(k for k in ck["model"] if ck["model"][k].dim() == 2)
    assert torch.allclose(ck["model"][k], (a[k] + b[k]) / 2, atol=1e-6)
    assert 0 < len(fin.reservoir) <= 8 and ck["reservoir"] is not None
    nxt = R.OfflineCLTrainer(-1, dicts, _opt(common + ["-finalize_only", "-load_from", name]), init_distributed=False)
    assert len(nxt.reservoir) == 0
    nxt.run(nxt._resume_checkpoint, [], valid)
    assert len(nxt.reservoir) == len(fin.reservoir)

"""Host-side logic of the distributed paths, run as gloo ranks on the CPU: the collective statement of the sharded
Adam(W) step against one process, a two-rank trainer end to end, a rank that disappears between steps, and the
heartbeat watchdog with an injected clock.  No GPU is involved and nothing here makes a device fault."""
import os
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port, timeout_s=60):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _spawn(worker, world, *args, timeout=240):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=timeout) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(results)


# ---------------------------------------------------------------------------------------------------------------
def _worker_sharded_adam(rank, world, port, q):
    try:
        _init(rank, world, port)
        from nmtgminor_b200.ops.reference import adamw_step
        from nmtgminor_b200.parallel.ddp import NcclReducer
        from nmtgminor_b200.parallel.symmetric import ShardedAdamReference
        total = 64 * world * 4
        torch.manual_seed(0)
        master = torch.randn(total)
        single_master = master.clone()
        m1, v1 = torch.zeros(total), torch.zeros(total)
        sharded = ShardedAdamReference(total, "cpu", weight_decay=0.01, max_grad_norm=1.0)
        worst = 0.0
        for step in range(1, 5):
            grads = [torch.randn(total, generator=torch.Generator().manual_seed(100 * step + r)) * 0.3 for r in range(world)]
            # one process sees the summed gradient
            adamw_step(single_master, sum(grads), m1, v1, lr=0.01, beta1=0.9, beta2=0.997, eps=1e-9, weight_decay=0.01, step=step,
                       grad_scale=0.5, max_grad_norm=1.0)
            mine = grads[rank].clone()
            norm = sharded.step(master, mine, lr=0.01, grad_scale=0.5)
            assert mine.abs().max() == 0                         # the step clears the gradient buffer
            assert abs(norm - float(sum(grads).norm()) * 0.5) < 1e-4 * norm
            worst = max(worst, (master - single_master).abs().max().item())
            # bucketed all-reduce == one all-reduce
            a, b = grads[rank].clone(), grads[rank].clone()
            NcclReducer(world)(a)
            NcclReducer(world, bucket_bytes=4 * 100)(b)
            assert torch.allclose(a, sum(grads), atol=1e-5) and torch.allclose(a, b, atol=1e-5)
        assert worst < 1e-5, worst
        q.put((rank, "ok", worst))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_adam_over_gloo_equals_one_process(world):
    for r in _spawn(_worker_sharded_adam, world):
        assert r[1] == "ok", r[2]


# ---------------------------------------------------------------------------------------------------------------
def _tiny_opt(extra=()):
    from nmtgminor_b200.options import default_options
    return default_options(["-model", "transformer", "-model_size", "64", "-layers", "1", "-n_heads", "2", "-inner_size", "128",
                            "-tie_weights", "-join_embedding", "-label_smoothing", "0.1", "-optim", "adam", "-learning_rate", "2e-3",
                            "-update_method", "regular", "-dropout", "0.1", "-batch_size_words", "256", "-log_interval", "1000",
                            "-seed", "3"] + list(extra))


def _corpus(n=96, vocab=120, seed=0):
    from nmtgminor_b200.data.dataset import Dataset
    from nmtgminor_b200.data.synthetic import synthetic_dict
    import numpy as np
    rng = np.random.RandomState(seed)
    src = [torch.from_numpy(rng.randint(4, vocab, size=rng.randint(5, 20)).astype("int64")) for _ in range(n)]
    tgt = [torch.from_numpy(np.concatenate([[2], rng.randint(4, vocab, size=rng.randint(5, 20)), [3]]).astype("int64")) for _ in range(n)]
    d = synthetic_dict(vocab)
    return Dataset(src, tgt, batch_size_words=256, multiplier=1), {"src": d, "tgt": d}


def _worker_trainer(rank, world, port, q, tmpdir):
    try:
        _init(rank, world, port)
        from nmtgminor_b200.train.trainer import Trainer
        data, dicts = _corpus()
        opt = _tiny_opt(["-save_model", os.path.join(tmpdir, "m"), "-epochs", "1", "-gpus", "-1"])
        opt.gpus = []
        os.environ["WORLD_SIZE"] = str(world)
        tr = Trainer(rank, dicts, opt, init_distributed=False)
        assert tr.world_size == world and tr.rank == rank
        before = [p.detach().clone() for p in tr.model.parameters()]
        last = tr.run(train_data=data, valid_data=data)
        moved = sum(float((a - b.detach()).abs().sum()) for a, b in zip(before, tr.model.parameters()))
        assert moved > 0
        # data parallel: identical parameters on every rank after training
        flat = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
        ref = flat.clone()
        dist.broadcast(ref, 0)
        assert torch.allclose(flat, ref, atol=1e-6), (flat - ref).abs().max()
        assert (last is not None) == (rank == 0)
        q.put((rank, "ok", moved))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_rank_trainer_on_cpu_keeps_the_ranks_in_step(tmp_path):
    for r in _spawn(_worker_trainer, 2, str(tmp_path)):
        assert r[1] == "ok", r[2]


# ---------------------------------------------------------------------------------------------------------------
def _worker_rank_leaves(rank, world, port, q):
    """Rank 1 leaves between steps (no collective of its own in flight).  The survivor's next collective must end
    with an error within the process-group timeout instead of hanging."""
    try:
        _init(rank, world, port, timeout_s=5)
        x = torch.ones(4)
        dist.all_reduce(x)                       # step 1: everybody is there
        assert float(x[0]) == world
        if rank == 1:
            dist.destroy_process_group()
            q.put((rank, "ok", "left"))
            return
        t0 = time.time()
        try:
            y = torch.ones(4)
            dist.all_reduce(y)                   # step 2: the peer is gone
            q.put((rank, "fail", "the collective returned although a rank had left"))
        except Exception as exc:  # noqa: BLE001 - any error is the expected outcome
            dt = time.time() - t0
            q.put((rank, "ok" if dt < 60 else "fail", "raised %s after %.1f s" % (type(exc).__name__, dt)))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))


def test_survivor_of_a_departed_gloo_rank_raises_instead_of_hanging():
    for r in _spawn(_worker_rank_leaves, 2, timeout=120):
        assert r[1] == "ok", r[2]


# ---------------------------------------------------------------------------------------------------------------
def test_heartbeat_reports_a_rank_that_stops_beating():
    from nmtgminor_b200.utils.watchdog import DictStore, Heartbeat, RankFailure
    now = [1000.0]
    clock = lambda: now[0]
    store = DictStore()
    a = Heartbeat(0, 2, timeout=10.0, store=store, clock=clock, start=False)
    b = Heartbeat(1, 2, timeout=10.0, store=store, clock=clock, start=False)
    for step in range(3):                        # both alive: publish and check by hand (the threads are not started)
        now[0] += 2.0
        a._publish()
        b._publish()
        assert a.check_peers() is None and b.check_peers() is None
        a.beat(step)
        b.beat(step)
    for _ in range(6):                           # rank 1 stops publishing; 12 s pass
        now[0] += 2.0
        a._publish()
    assert a.check_peers() == 1
    a.failed = a.check_peers()                   # what the background loop does
    with pytest.raises(RankFailure):
        a.beat(4)
    assert b.check_peers() is None               # rank 0 kept beating


def test_heartbeat_thread_notices_a_silent_peer_in_real_time():
    from nmtgminor_b200.utils.watchdog import DictStore, Heartbeat, RankFailure
    store = DictStore()
    seen = []
    a = Heartbeat(0, 2, timeout=0.3, interval=0.05, store=store, on_failure=lambda r, t: seen.append(r))
    b = Heartbeat(1, 2, timeout=0.3, interval=0.05, store=store)
    time.sleep(0.2)
    assert a.failed is None
    b.stop()                                     # rank 1 goes silent
    deadline = time.time() + 5.0
    while a.failed is None and time.time() < deadline:
        time.sleep(0.05)
    a.stop()
    assert a.failed == 1 and seen == [1]
    with pytest.raises(RankFailure):
        a.beat(1)


# ---------------------------------------------------------------------------------------------------------------
def test_resume_continues_exactly_where_the_uninterrupted_run_would_be(tmp_path):
    """12 updates in one go == 6 updates, save, restore in a fresh trainer, 6 more: bitwise on the CPU (parameters,
    optimiser moments, update count, learning rate, dropout masks, batch order)."""
    sys.path.insert(0, ROOT)
    from nmtgminor_b200.train.checkpoint import load_checkpoint
    from nmtgminor_b200.train.trainer import Trainer

    def trainer(extra):
        torch.manual_seed(0)
        data, dicts = _corpus(n=160)
        opt = _tiny_opt(["-epochs", "1", "-update_method", "noam", "-warmup_steps", "8", "-learning_rate", "1.0"] + extra)
        opt.gpus = []
        return Trainer(0, dicts, opt, init_distributed=False), data

    full, data = trainer(["-save_model", str(tmp_path / "full"), "-max_step", "12"])
    full.run(train_data=data, valid_data=None)
    assert full.optim._step == 12

    first, data = trainer(["-save_model", str(tmp_path / "part"), "-max_step", "6", "-save_every", "6"])
    first.run(train_data=data, valid_data=None)
    files = sorted(str(p) for p in tmp_path.glob("part_ppl_*_e0.*.pt"))
    assert files, list(tmp_path.iterdir())
    ckpt = load_checkpoint(files[0])
    assert ckpt["optim"]["_step"] == 6 and ckpt["itr"] is not None

    second, data = trainer(["-save_model", str(tmp_path / "resumed"), "-max_step", "12", "-load_from", files[0]])
    assert second.optim._step == 6
    assert abs(second.optim.current_lr() - first.optim.current_lr()) < 1e-12
    second.run(train_data=data, valid_data=None)
    assert second.optim._step == 12
    for (n, a), (_, b) in zip(full.model.named_parameters(), second.model.named_parameters()):
        assert torch.equal(a, b), "parameter %s differs after resume (max %g)" % (n, (a - b).abs().max())
    sa, sb = full.optim.optimizer.state_dict()["state"], second.optim.optimizer.state_dict()["state"]
    for k in sa:
        assert torch.equal(sa[k]["exp_avg"], sb[k]["exp_avg"]) and torch.equal(sa[k]["exp_avg_sq"], sb[k]["exp_avg_sq"])

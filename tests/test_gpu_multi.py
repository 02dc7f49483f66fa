"""Peer-memory data parallelism on real GPUs: the fused reduce-scatter + Adam(W) + all-gather kernels against the
collective-based statement of the same step, the bounded-wait timeout path, and a short 2-GPU training run."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))


def _worker_fused_vs_reference(rank, world, port, q):
    try:
        _init(rank, world, port)
        from nmtgminor_b200 import ops
        from nmtgminor_b200.options import default_options
        from nmtgminor_b200.parallel.flat import FlatParameterStore
        from nmtgminor_b200.parallel.symmetric import FusedAllReduceAdam, ShardedAdamReference, SymmetricHeap
        from nmtgminor_b200.train.optim import Optim
        dev = torch.device("cuda", rank)
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(256, 1024), torch.nn.Linear(1024, 512), torch.nn.Linear(512, 64)).to(dev)
        heap = SymmetricHeap(dev)
        ptrs = {}

        def symm(name):
            def alloc(n, dt):
                t, p = heap.alloc(n, dt)
                ptrs[name] = p
                return t
            return alloc
        store = FlatParameterStore(model, dev, allocator={"grad": symm("grad"), "work": symm("work")}, pad_total_to=256 * world)
        opt = default_options(["-optim", "adam", "-learning_rate", "0.01", "-update_method", "regular", "-weight_decay", "0.01",
                               "-max_grad_norm", "1.0"])
        optim = Optim(opt)
        optim.set_parameters(model.parameters(), store)
        fused = FusedAllReduceAdam(store, optim, heap, ptrs["grad"], ptrs["work"])
        optim.attach_distributed(fused)
        ref_master = store.master.clone()
        ref = ShardedAdamReference(store.total, dev, weight_decay=0.01, max_grad_norm=1.0)
        worst = 0.0
        for step in range(1, 4):
            g = torch.Generator(device=dev).manual_seed(100 * step + rank)
            grad = torch.randn(store.total, device=dev, generator=g) * 0.05
            store.grad.copy_(grad)
            ref_grad = grad.clone()
            optim._step += 1
            optim.write_hyper(0.5)
            fused(store.grad)          # end of a backward pass: reduce every unit
            optim.launch_fused()
            norm_ref = ref.step(ref_master, ref_grad, lr=0.01, grad_scale=0.5)
            torch.cuda.synchronize()
            dist.barrier()
            assert ops.check_status() == 0
            fused.gather_master()
            err = (store.master - ref_master).abs().max().item()
            worst = max(worst, err)
            assert err < 2e-5, "master mismatch %g at step %d" % (err, step)
            assert (store.work.float() - ref_master).abs().max().item() < 2e-2
            assert store.grad.abs().max().item() == 0.0
            assert abs(fused.norm.item() - norm_ref) / norm_ref < 1e-3
        q.put((rank, "ok", worst))
    except Exception as exc:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(worker, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1] == "ok", "rank %d failed:\n%s" % (r[0], r[2])
    return results


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allreduce_adam_matches_collectives(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    _run(_worker_fused_vs_reference, world)


def test_peer_wait_times_out_without_hanging():
    """A wait on a flag nobody raises must give up, record the status, and leave the context usable."""
    from nmtgminor_b200 import ops
    dev = torch.device("cuda", 0)
    flags = torch.zeros(3 * 16, dtype=torch.int32, device=dev)
    ops.check_status()
    before = ops.ext().get_peer_timeout_ms()
    ops.ext().set_peer_timeout_ms(300.0)
    try:
        ops.ext().peer_wait_row(0, [flags.data_ptr(), flags.data_ptr()], 0, 7, flags)   # slot 1 is never written
        torch.cuda.synchronize()
    finally:
        ops.ext().set_peer_timeout_ms(before)
    assert ops.check_status() == 5
    x = torch.ones(4, device=dev)
    assert float((x + 1).sum()) == 8.0


def _worker_train(rank, world, port, q):
    try:
        _init(rank, world, port)
        from nmtgminor_b200 import ops
        from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
        from nmtgminor_b200.models.transformer import Transformer
        from nmtgminor_b200.options import default_options
        from nmtgminor_b200.train.engine import TrainEngine
        torch.manual_seed(1)
        opt = default_options(["-model_size", "256", "-layers", "2", "-n_heads", "4", "-inner_size", "1024", "-tie_weights",
                               "-join_embedding", "-ffn_activation", "relu", "-label_smoothing", "0.1", "-optim", "adam",
                               "-learning_rate", "1e-3", "-update_method", "regular", "-dropout", "0.1", "-weight_decay", "0.01"])
        d = synthetic_dict(2000)
        model = Transformer(opt, {"src": d, "tgt": d})
        eng = TrainEngine(model, opt, device="cuda:%d" % rank, cuda_graph=True, ddp="fused")
        assert getattr(eng.optim, "distributed", None) is not None, "fused reducer was not attached"
        batches = [b.pin_memory() for b in token_budget_batches(2000, 5, 40, 1024, 4, seed=5 + rank, static=True)]
        first = last = None
        for it in range(30):
            b = batches[it % len(batches)]
            loss, _ = eng.train_step(b)
            v = loss.item() / b.tgt_size
            first = v if first is None else first
            last = v
        torch.cuda.synchronize()
        assert ops.check_status() == 0
        assert last < first - 0.5, (first, last)
        # all ranks hold identical parameters after the peer all-gather
        w = eng.store.work.float()
        ref = w.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(w, ref)
        q.put((rank, "ok", last))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_gpu_training_with_fused_ddp():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(_worker_train, 2)


def _small_opt(extra=()):
    from nmtgminor_b200.options import default_options
    return default_options(["-model_size", "256", "-layers", "3", "-n_heads", "4", "-inner_size", "1024", "-tie_weights",
                            "-join_embedding", "-ffn_activation", "relu", "-label_smoothing", "0.1", "-optim", "adam",
                            "-learning_rate", "1e-3", "-update_method", "regular", "-dropout", "0.0", "-attn_dropout", "0.0",
                            "-emb_dropout", "0.0", "-weight_decay", "0.01"] + list(extra))


def _train_losses(ddp, rank, steps=8, seed_off=0, graph=False):
    from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
    from nmtgminor_b200.models.transformer import Transformer
    from nmtgminor_b200.train.engine import TrainEngine
    torch.manual_seed(1)
    d = synthetic_dict(2000)
    model = Transformer(_small_opt(), {"src": d, "tgt": d})
    eng = TrainEngine(model, _small_opt(), device="cuda:%d" % rank, cuda_graph=graph, ddp=ddp)
    batches = [b.pin_memory() for b in token_budget_batches(2000, 5, 40, 1024, 4, seed=5 + seed_off, static=True)]
    losses = []
    for it in range(steps):
        loss, _ = eng.train_step(batches[it % len(batches)])
        losses.append(loss.item())
    torch.cuda.synchronize()
    return eng, losses


def test_fsdp_single_rank_matches_plain_engine():
    """World size 1 exercises the whole sharded path (units, staging buffers, gather hooks, sharded Adam)."""
    from nmtgminor_b200 import ops
    _, plain = _train_losses(None, 0)
    eng, sharded = _train_losses("fsdp", 0)
    assert ops.check_status() == 0
    fs = eng.optim.distributed
    assert len([u for u in fs.units if u.slot >= 0]) == 6 and fs.store.work is None
    for a, b in zip(plain, sharded):
        assert abs(a - b) < 2e-3 * abs(a), (plain, sharded)
    assert sharded[-1] < sharded[0]
    fs.gather_master()
    assert torch.isfinite(eng.store.master).all()


def _worker_fsdp(rank, world, port, q):
    try:
        _init(rank, world, port)
        from nmtgminor_b200 import ops
        eng_f, fused = _train_losses("fused", rank, seed_off=rank)
        eng_s, sharded = _train_losses("fsdp", rank, seed_off=rank)
        assert ops.check_status() == 0
        for a, b in zip(fused, sharded):
            assert abs(a - b) < 5e-3 * abs(a), (fused, sharded)
        # the sharded master weights, gathered, equal the data-parallel run's weights
        eng_f.optim.distributed.gather_master()
        eng_s.optim.distributed.gather_master()
        # Adam moves every weight by about lr per step, so rounding-level gradient differences can flip single steps
        delta = (eng_f.store.master - eng_s.store.master).abs()
        assert delta.max().item() < 2e-2 and delta.mean().item() < 2e-4, (delta.max().item(), delta.mean().item())
        eng_s.optim.distributed.release_master()
        rep = eng_s.optim.distributed.memory_report()
        assert rep["bf16_shard"] * world <= rep["replicated_bf16_would_be"] * 1.05 + 4096 * world
        # what survives a step per parameter: bf16 + fp32 master + reduced gradient + two moments, all 1 / world
        assert rep["persistent_bytes_per_param"] <= 18.0 / world * 1.05 + 1e-3, rep
        assert not rep["full_master_resident"]
        q.put((rank, "ok", sharded[-1]))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fsdp_matches_fused_data_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    _run(_worker_fsdp, world)


def test_fsdp_single_rank_under_cuda_graph_and_unfused_gather_agree():
    """The captured step (gathers inside the GEMMs, per-layer reductions on the communication stream as fork / join
    edges of the graph) and the eager step with the stand-alone copy kernel train the same model."""
    import os
    from nmtgminor_b200 import ops
    _, graphed = _train_losses("fsdp", 0, graph=True)
    os.environ["NMTG_FSDP_FUSED_GATHER"] = "0"
    try:
        _, unfused = _train_losses("fsdp", 0)
    finally:
        del os.environ["NMTG_FSDP_FUSED_GATHER"]
    assert ops.check_status() == 0
    for a, b in zip(graphed, unfused):
        assert abs(a - b) < 2e-3 * abs(a), (graphed, unfused)
    assert graphed[-1] < graphed[0]


def _worker_resume(rank, world, port, q, ddp, tmpdir):
    """Train 3 steps, save, 3 more; a second engine restores the file and must reproduce steps 4-6 on every rank."""
    try:
        _init(rank, world, port)
        from nmtgminor_b200 import ops
        from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
        from nmtgminor_b200.models.transformer import Transformer
        from nmtgminor_b200.train.checkpoint import load_checkpoint, load_model_state, model_state_for_saving
        from nmtgminor_b200.train.engine import TrainEngine
        d = synthetic_dict(2000)
        batches = [b.pin_memory() for b in token_budget_batches(2000, 5, 40, 1024, 6, seed=11 + rank, static=True)]

        def build():
            torch.manual_seed(1)
            model = Transformer(_small_opt(), {"src": d, "tgt": d})
            return model, TrainEngine(model, _small_opt(), device="cuda:%d" % rank, cuda_graph=False, ddp=ddp)

        model, eng = build()
        for it in range(3):
            eng.train_step(batches[it])
        dist_opt = eng.optim.distributed
        dist_opt.gather_master()
        eng.optim.prepare_state_dict()
        path = os.path.join(tmpdir, "ckpt.pt")
        if rank == 0:
            torch.save({"model": model_state_for_saving(model), "optim": eng.optim.state_dict()}, path)
        if hasattr(dist_opt, "release_master"):
            dist_opt.release_master()
        dist.barrier()
        want = [eng.train_step(batches[it])[0].item() for it in range(3, 6)]
        torch.cuda.synchronize()
        dist.barrier()
        ckpt = load_checkpoint(path)
        model2 = Transformer(_small_opt(), {"src": d, "tgt": d})
        load_model_state(model2, ckpt["model"])
        eng2 = TrainEngine(model2, _small_opt(), device="cuda:%d" % rank, cuda_graph=False, ddp=ddp)
        eng2.optim.load_state_dict(ckpt["optim"])
        assert eng2.optim._step == 3
        got = [eng2.train_step(batches[it])[0].item() for it in range(3, 6)]
        torch.cuda.synchronize()
        assert ops.check_status() == 0
        for a, b in zip(want, got):
            assert abs(a - b) < 1e-3 * abs(a), (rank, want, got)
        # every rank got its moments back (the failure this guards against: only rank 0's slice being saved)
        m1, m2 = eng.optim.distributed.exp_avg, eng2.optim.distributed.exp_avg
        assert m2.abs().sum().item() > 0
        q.put((rank, "ok", got[-1]))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run_args(worker, world, *args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1] == "ok", "rank %d failed:\n%s" % (r[0], r[2])
    return results


@pytest.mark.parametrize("ddp", ["fused", "fsdp"])
def test_two_gpu_save_and_resume_restores_every_ranks_optimizer_state(ddp, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run_args(_worker_resume, 2, ddp, str(tmp_path))

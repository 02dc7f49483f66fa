"""Headline benchmark: training throughput (target tokens / s) of Transformer-big, bf16, data parallel.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config big|tiny_cpu]

Model / data (the reference's own headline setting for NMT training): 6 + 6 layers, d_model 1024, 16
heads, FFN 4096 ReLU, dropout 0.1, shared 32000-word vocabulary with tied embeddings / output layer, AdamW,
label-smoothed cross-entropy.  Every GPU draws a pool of sentence pairs with lengths uniform in [20, 100]
and uniform random token ids (synthetic: no data set is reachable) and cuts it into batches with the
reference's own rule (onmt/data/dataset.py:862-953, onmt/data/batch_utils.py:7-59): sort by (target, source)
length, fill a batch while ``max(length) * (sentences + 1) <= batch_size_words``, trim to a multiple of 8
sentences.  ``batch_size_words`` is 13000, which gives 8.2 k real target tokens per batch on average (2.8 k to
12.9 k; targets 99.7 % full, sources 64 % full when padded).  BOTH arms step through the same batches: this
framework packs them (no padding positions), the reference pads them as its collate function does.
Weak scaling: per-GPU work is fixed, the reported value is the sum over GPUs; in every step all ranks take the
batch of the same length quantile from their own pool, so no rank waits for a longer batch of another.

For N > 1 the script is launched once per GPU by ``python -m torch.distributed.run`` and reads
RANK / LOCAL_RANK / WORLD_SIZE from the environment.  Rank 0 prints ONE JSON line.

Measurements per run, all bracketed by a barrier + device synchronisation and timed with CUDA events (max
over ranks):
* ``value``: K steps back to back; the loss stays on the device.
* ``e2e``:   K steps through the public step call where every step also copies its inputs from pinned host
  memory and reads its loss back to the host.
* ``exposed_comm_ms`` (N > 1, this framework's arm): ms per step minus ms per step of the same steps with the
  gradient exchange replaced by a local optimiser update on every rank (the ranks' parameters diverge in that
  run, so it comes last).  ``comm_roofline_ms`` is what the step's NVLink traffic would take at the measured
  770 GB/s per direction if none of it were hidden.
The working set of a step (weights, optimiser state, activations: several GB) is far larger than the 126 MB
L2, so no explicit flush is needed between iterations.

``--config tiny_cpu`` runs the 2 + 2 layer, d_model 256 model on the CPU in fp32 (batches of 32 sentence pairs,
lengths uniform in [10, 50]) for both arms, timed with the wall clock.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

VOCAB = 32000
BATCH_SIZE_WORDS = 13000      # padded positions per batch under the reference's rule: 8.2 k real target tokens on average
POOL_SENTENCES = 20000
MIN_LEN, MAX_LEN = 20, 100
N_DISTINCT_BATCHES = 8
NVLINK_GBS = 770.0            # measured peer-copy bandwidth per direction on this pool


# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.strip().split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()       # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_rule_batches(lengths, order, batch_size_words, multiplier=8):
    """Greedy token-budget batches, the rule of the reference's ``allocate_batch`` (onmt/data/batch_utils.py:7-59):
    a batch is closed when ``max(length) * (sentences + 1)`` would exceed the budget and trimmed to a multiple of
    ``multiplier`` sentences (the remainder opens the next batch)."""
    batches, cur, sizes = [], [], []
    for i in order:
        if cur and max(max(sizes), lengths[i]) * (len(cur) + 1) > batch_size_words:
            n = len(cur)
            keep = max(multiplier * (n // multiplier), n % multiplier)
            batches.append(cur[:keep])
            cur, sizes = cur[keep:], sizes[keep:]
        cur.append(int(i))
        sizes.append(int(lengths[i]))
    if cur:
        batches.append(cur)
    return batches


def sentence_groups(n_groups: int, seed: int, min_len=MIN_LEN, max_len=MAX_LEN, vocab=VOCAB, pool=POOL_SENTENCES,
                    batch_size_words=BATCH_SIZE_WORDS, batch_size_sents=None):
    """``n_groups`` batches (lists of source / target id tensors) spread evenly over the length-sorted batch list of
    one synthetic pool, visited in a fixed scrambled order so that consecutive steps differ in length."""
    rng = np.random.RandomState(seed)
    src_len = rng.randint(min_len, max_len + 1, size=pool)
    tgt_len = rng.randint(min_len, max_len + 1, size=pool) + 2            # BOS ... EOS
    if batch_size_sents is None:
        order = np.lexsort((src_len, tgt_len))                              # the reference's order for text corpora
        lengths = np.maximum(src_len, tgt_len - 1)
        batches = reference_rule_batches(lengths, order, batch_size_words)
    else:                                                                   # fixed sentence count, unsorted (config 1)
        batches = [list(range(k, k + batch_size_sents)) for k in range(0, pool - batch_size_sents + 1, batch_size_sents)]
    pick = [batches[int(round(q * (len(batches) - 2)))] for q in np.linspace(0.0, 1.0, n_groups)]
    scramble = [(5 * k + 3) % n_groups for k in range(n_groups)] if n_groups % 5 else list(range(n_groups))
    groups = []
    for k in scramble:
        src = [torch.from_numpy(rng.randint(4, vocab, size=src_len[i]).astype(np.int64)) for i in pick[k]]
        tgt = [torch.from_numpy(np.concatenate([[2], rng.randint(4, vocab, size=tgt_len[i] - 2), [3]]).astype(np.int64)) for i in pick[k]]
        groups.append((src, tgt))
    return groups


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def timed_loop(step_fn, batches, tokens, steps, world, read_loss: bool):
    """Returns (milliseconds for `steps` steps [max over ranks], target tokens of this rank)."""
    barrier(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ntok = 0
    ev0.record()
    for i in range(steps):
        loss = step_fn(batches[i % len(batches)])
        ntok += tokens[i % len(batches)]
        if read_loss:
            _ = float(loss)            # device -> host read of the step's result
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    barrier(world)
    return max_over_ranks(ms, world), ntok


# ---------------------------------------------------------------------------------------------------
MODEL_NAME = "transformer-big 6+6 d1024 h16 ffn4096 relu vocab32000 tied"


def result_line(impl, world, args, ms, ntok_total, ms_e2e, ntok_e2e_total, h2d, n_params, clocks, details, extra=None):
    """One JSON object in the driver's format; ``config`` holds only what both arms share."""
    out = {
        "metric": "train target tokens/s", "value": ntok_total / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": impl,
        "config": {"model": MODEL_NAME, "global_batch": int(round(ntok_total / args.steps)), "global_batch_unit": "target tokens",
                   "seq_len": "uniform[20,100]", "parallelism": "dp%d" % world, "optimizer": "adamw", "params": n_params,
                   "batching": "length-sorted, max(len)*(n+1) <= %d, multiples of 8 sentences (the reference's rule); same "
                               "batches for both arms" % BATCH_SIZE_WORDS,
                   "l2": "per-step working set (weights + optimizer state + activations, several GB) exceeds the 126 MB L2; no flush"},
        "impl_details": details,
        "clocks": clocks,
        "e2e": {"value": ntok_e2e_total / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
    }
    out.update(extra or {})
    return out


def run_ours(args, rank, local, world):
    from nmtgminor_b200 import ops
    from nmtgminor_b200.data.dataset import collate
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.models.transformer import Transformer
    from nmtgminor_b200.options import default_options
    from nmtgminor_b200.train.engine import TrainEngine

    ops.ext()   # fail loudly when the sm_100a extension is missing
    torch.manual_seed(1234)
    opt = default_options(["-model", "transformer", "-layers", "6", "-model_size", "1024", "-n_heads", "16", "-inner_size", "4096",
                           "-dropout", "0.1", "-attn_dropout", "0.1", "-emb_dropout", "0.1", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding", "-label_smoothing", "0.1", "-optim", "adam", "-weight_decay", "0.01",
                           "-learning_rate", "2.0", "-update_method", "noam", "-warmup_steps", "4000", "-max_grad_norm", "5",
                           "-fp16", "-bf16", "-batch_size_words", str(BATCH_SIZE_WORDS)])
    d = synthetic_dict(VOCAB)
    model = Transformer(opt, {"src": d, "tgt": d})
    n_params = sum(p.numel() for p in model.parameters())
    ddp = args.ddp if (world > 1 or args.ddp == "fsdp") else None
    engine = TrainEngine(model, opt, device="cuda:%d" % local, cuda_graph=not args.no_graph, ddp=ddp)

    groups = sentence_groups(N_DISTINCT_BATCHES, seed=1000 + rank)
    # packed (padding-free) batches; capacities rounded to shape classes, one captured graph per class
    batches = [collate(src, tgt, padded=False, packed=True, static_shapes=True).pin_memory() for src, tgt in groups]
    tokens = [b.tgt_size for b in batches]
    h2d = int(np.mean([b.h2d_bytes(hot_only=True) for b in batches]))

    step = lambda b: engine.train_step(b)[0]
    # every shape class once kernel by kernel (which also captures its graph) and once replayed, then the W warm-up steps
    for _ in range(2):
        for b in batches:
            loss = step(b)
    for i in range(args.warmup):
        loss = step(batches[i % len(batches)])
    first_loss = float(loss) / tokens[(args.warmup - 1) % len(batches)]
    # kernels of this framework enqueued per step (counted by the op layer; a graph replays the captured set)
    launches_per_step = engine.kernel_launches_per_step

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, ntok = timed_loop(step, batches, tokens, args.steps, world, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, ntok_e2e = timed_loop(step, batches, tokens, args.steps, world, read_loss=True)
    status = ops.check_status()
    extra = {"gpu_launches": (launches_per_step or 0) * args.steps, "gpu_launches_per_step": launches_per_step,
             "kernel_status": status, "loss_per_token_after_warmup": first_loss}
    if world > 1 and ddp in ("fused", "fsdp") and not args.no_exposed:
        # the same steps without the gradient exchange: every rank updates its own full copy locally
        engine.local_only_mode()
        for _ in range(2):
            for b in batches:
                step(b)
        ms_local, _ = timed_loop(step, batches, tokens, args.steps, world, read_loss=False)
        p_bytes = float(n_params)
        nv_ms = ((world - 1) / world * p_bytes * 4 + (world - 1) / world * p_bytes * 2) / (NVLINK_GBS * 1e9) * 1e3
        extra.update({"exposed_comm_ms": (ms - ms_local) / args.steps, "ms_per_step_without_exchange": ms_local / args.steps,
                      "comm_roofline_ms": nv_ms,
                      "comm_bytes_per_rank_per_step": {"in": (world - 1) / world * p_bytes * 4, "out": (world - 1) / world * p_bytes * 2}})
    total_tok = sum_over_ranks(float(ntok), world)
    total_tok_e2e = sum_over_ranks(float(ntok_e2e), world)
    if rank == 0:
        details = {"cuda_graph": not args.no_graph, "ddp": ddp, "graphs_captured": len(engine._graphs),
                   "path": "packed batches, tcgen05 kernels, flat AdamW" + (", peer-memory reduce overlapped with backward" if ddp == "fused" else "")}
        print(json.dumps(result_line("ours", world, args, ms, total_tok, ms_e2e, total_tok_e2e, h2d, n_params, clocks, details, extra)),
              flush=True)


def run_reference(args, rank, local, world):
    from bench_reference import ReferenceRunner, reference_available
    ok, why = reference_available()
    if not ok:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return
    torch.manual_seed(1234)
    try:
        runner = ReferenceRunner(VOCAB, "cuda:%d" % local, rank, world)
    except Exception as exc:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference failed to build: %r" % (exc,)}), flush=True)
        return
    groups = sentence_groups(N_DISTINCT_BATCHES, seed=1000 + rank)
    batches = [runner.collate(s, t) for s, t in groups]
    tokens = [int(b.tensors["tgt_size"]) for b in batches]
    h2d = int(np.mean([runner.h2d_bytes(b) for b in batches]))
    step = runner.step
    for b in batches:                       # every batch shape once (allocator, cuBLAS heuristics), then the W warm-up steps
        loss = step(b)
    for i in range(args.warmup):
        loss = step(batches[i % len(batches)])
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, ntok = timed_loop(step, batches, tokens, args.steps, world, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, ntok_e2e = timed_loop(step, batches, tokens, args.steps, world, read_loss=True)
    total_tok = sum_over_ranks(float(ntok), world)
    total_tok_e2e = sum_over_ranks(float(ntok_e2e), world)
    if rank == 0:
        details = {"path": "autocast bf16 + GradScaler + DistributedDataParallel(NCCL), padded batches from the reference's collate_fn"}
        print(json.dumps(result_line("reference", world, args, ms, total_tok, ms_e2e, total_tok_e2e, h2d, runner.n_params, clocks, details,
                                     {"gpu_launches": 0})), flush=True)


# ---------------------------------------------------------------------------------------------------
# config 1: tiny Transformer on the CPU, fp32, both arms
# ---------------------------------------------------------------------------------------------------
def run_tiny_cpu(args):
    torch.manual_seed(1)
    vocab = 8000
    groups = sentence_groups(8, seed=1, min_len=10, max_len=50, vocab=vocab, pool=2048, batch_size_sents=32)
    if args.impl == "reference":
        from bench_reference import ReferenceRunner, reference_available
        ok, why = reference_available()
        if not ok:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
            return
        runner = ReferenceRunner(vocab, "cpu", tiny=True, argv_extra=["-optim", "adam", "-learning_rate", "1e-3", "-update_method", "regular",
                                                                      "-weight_decay", "0.0"])
        batches = [runner.collate(s, t) for s, t in groups]
        tokens = [int(b.tensors["tgt_size"]) for b in batches]
        step = lambda b: float(runner.step(b))
        n_params = runner.n_params
    else:
        from nmtgminor_b200.data.dataset import collate
        from nmtgminor_b200.data.synthetic import synthetic_dict
        from nmtgminor_b200.models.transformer import Transformer
        from nmtgminor_b200.options import default_options
        from nmtgminor_b200.train.engine import TrainEngine
        opt = default_options(["-model", "transformer", "-layers", "2", "-model_size", "256", "-n_heads", "4", "-inner_size", "1024",
                               "-dropout", "0.1", "-attn_dropout", "0.1", "-emb_dropout", "0.1", "-ffn_activation", "relu", "-tie_weights",
                               "-join_embedding", "-label_smoothing", "0.1", "-optim", "adam", "-learning_rate", "1e-3",
                               "-update_method", "regular", "-max_grad_norm", "5"])
        d = synthetic_dict(vocab)
        model = Transformer(opt, {"src": d, "tgt": d})
        engine = TrainEngine(model, opt, device="cpu")
        batches = [collate(s, t, padded=False, packed=True) for s, t in groups]
        tokens = [b.tgt_size for b in batches]
        step = lambda b: float(engine.train_step(b)[0])
        n_params = sum(p.numel() for p in model.parameters())
    for i in range(args.warmup):
        step(batches[i % len(batches)])
    t0 = time.perf_counter()
    ntok = 0
    for i in range(args.steps):
        step(batches[i % len(batches)])
        ntok += tokens[i % len(batches)]
    dt = time.perf_counter() - t0
    print(json.dumps({
        "metric": "train target tokens/s", "value": ntok / dt, "unit": "tokens/s", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "impl": args.impl,
        "config": {"model": "tiny transformer 2+2 d256 h4 ffn1024 relu vocab8000 tied", "global_batch": int(round(ntok / args.steps)),
                   "global_batch_unit": "target tokens", "seq_len": "uniform[10,50]", "parallelism": "cpu", "optimizer": "adam",
                   "params": n_params, "batching": "32 sentence pairs per batch, unsorted", "threads": torch.get_num_threads()},
        "timing": "wall clock (CPU run; loss read every step)", "gpu_launches": 0}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="big", choices=["big", "tiny_cpu"])
    ap.add_argument("--ddp", default="fused", choices=["fused", "nccl", "fsdp"],
                    help="N > 1: peer-memory reduction fused with the optimiser, NCCL all-reduce, or fully sharded parameters")
    ap.add_argument("--no-graph", action="store_true", help="run the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-exposed", action="store_true", help="skip the extra run that measures the exposed communication time")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.config == "tiny_cpu":
        run_tiny_cpu(args)
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    rank, local, world = dist_setup(args.gpus)
    try:
        if args.impl == "reference":
            run_reference(args, rank, local, world)
        else:
            run_ours(args, rank, local, world)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

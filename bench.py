"""Headline benchmark: training throughput (target tokens / s) of Transformer-big, bf16, data parallel.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

Model / data (the reference's own headline setting for NMT training): 6 + 6 layers, d_model 1024, 16
heads, FFN 4096 ReLU, dropout 0.1, shared 32000-word vocabulary with tied embeddings / output layer, AdamW,
label-smoothed cross-entropy; every GPU gets batches of ~8192 real target tokens built from sentence pairs
with lengths uniform in [20, 100] and uniform random token ids (synthetic: no data set is reachable).
Weak scaling: per-GPU work is fixed, the reported value is the sum over GPUs.

For N > 1 the script is launched once per GPU by ``python -m torch.distributed.run`` and reads
RANK / LOCAL_RANK / WORLD_SIZE from the environment.  Rank 0 prints ONE JSON line.

Two measurements per run, both bracketed by a barrier + device synchronisation and timed with CUDA events
(max over ranks):
* ``value``: K steps back to back; the loss stays on the device.
* ``e2e``:   K steps through the public step call where every step also copies its inputs from pinned host
  memory and reads its loss back to the host.
The working set of a step (weights, optimiser state, activations: several GB) is far larger than the 126 MB
L2, so no explicit flush is needed between iterations.
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
TOKENS_PER_GPU = 8192
MIN_LEN, MAX_LEN = 20, 100
N_DISTINCT_BATCHES = 8


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
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
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


def sentence_groups(n_groups: int, seed: int):
    """Groups of (source, target) id tensors with ~TOKENS_PER_GPU real target tokens each."""
    rng = np.random.RandomState(seed)
    groups = []
    for _ in range(n_groups):
        src, tgt, tot = [], [], 0
        while True:
            ls, lt = rng.randint(MIN_LEN, MAX_LEN + 1), rng.randint(MIN_LEN, MAX_LEN + 1)
            if tot + lt + 1 > TOKENS_PER_GPU and tgt:
                break
            src.append(torch.from_numpy(rng.randint(4, VOCAB, size=ls).astype(np.int64)))
            tgt.append(torch.from_numpy(np.concatenate([[2], rng.randint(4, VOCAB, size=lt), [3]]).astype(np.int64)))
            tot += lt + 1
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
                           "-fp16", "-bf16", "-batch_size_words", str(TOKENS_PER_GPU)])
    d = synthetic_dict(VOCAB)
    model = Transformer(opt, {"src": d, "tgt": d})
    n_params = sum(p.numel() for p in model.parameters())
    engine = TrainEngine(model, opt, device="cuda:%d" % local, cuda_graph=not args.no_graph,
                         ddp=(args.ddp if (world > 1 or args.ddp == "fsdp") else None))

    groups = sentence_groups(N_DISTINCT_BATCHES, seed=1000 + rank)
    up = lambda v: (v + 127) // 128 * 128
    cap_s = up(max(sum(len(s) for s in g[0]) for g in groups))
    cap_t = up(max(sum(len(t) - 1 for t in g[1]) for g in groups))
    max_b = max(len(g[0]) for g in groups)
    batches = []
    for src, tgt in groups:
        b = collate(src, tgt, padded=False, packed=True, capacity_src=cap_s, capacity_tgt=cap_t, max_batch=max_b)
        b.packed_source().max_len = MAX_LEN
        b.packed_target_input().max_len = MAX_LEN + 1
        batches.append(b.pin_memory())
    tokens = [b.tgt_size for b in batches]
    h2d = int(np.mean([b.h2d_bytes(hot_only=True) for b in batches]))

    step = lambda b: engine.train_step(b)[0]
    for i in range(args.warmup):
        loss = step(batches[i % len(batches)])
    first_loss = float(loss) / tokens[(args.warmup - 1) % len(batches)] if args.warmup else None
    # kernels of this framework enqueued per step (counted by the op layer; a graph replays the captured set)
    launches_per_step = engine.kernel_launches_per_step

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, ntok = timed_loop(step, batches, tokens, args.steps, world, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, ntok_e2e = timed_loop(step, batches, tokens, args.steps, world, read_loss=True)
    status = ops.check_status()
    total_tok = sum_over_ranks(float(ntok), world)
    total_tok_e2e = sum_over_ranks(float(ntok_e2e), world)
    if rank == 0:
        value = total_tok / (ms / 1e3)
        out = {
            "metric": "train target tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": "transformer-big 6+6 d1024 h16 ffn4096 relu vocab32000 tied", "global_batch": int(round(total_tok / args.steps)),
                       "global_batch_unit": "target tokens", "seq_len": "uniform[20,100]", "parallelism": "dp%d" % world,
                       "optimizer": "adamw", "params": n_params, "cuda_graph": not args.no_graph, "ddp": args.ddp if (world > 1 or args.ddp == "fsdp") else None,
                       "l2": "per-step working set (weights + optimizer state + activations, several GB) exceeds the 126 MB L2; no flush"},
            "clocks": clocks,
            "e2e": {"value": total_tok_e2e / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": (launches_per_step or 0) * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "kernel_status": status, "loss_per_token_after_warmup": first_loss,
        }
        print(json.dumps(out), flush=True)


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
        out = {
            "metric": "train target tokens/s", "value": total_tok / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": "transformer-big 6+6 d1024 h16 ffn4096 relu vocab32000 tied", "global_batch": int(round(total_tok / args.steps)),
                       "global_batch_unit": "target tokens", "seq_len": "uniform[20,100]", "parallelism": "dp%d" % world,
                       "optimizer": "adamw", "params": runner.n_params, "path": "autocast bf16 + GradScaler + DistributedDataParallel(NCCL)",
                       "l2": "per-step working set exceeds the 126 MB L2; no flush"},
            "clocks": clocks,
            "e2e": {"value": total_tok_e2e / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0,
        }
        print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ddp", default="fused", choices=["fused", "nccl", "fsdp"],
                    help="N > 1: peer-memory reduction fused with the optimiser, NCCL all-reduce, or fully sharded parameters")
    ap.add_argument("--no-graph", action="store_true", help="run the step eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
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

"""Micro-benchmark of the peer-memory communication kernels on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_comm.py [--params 209e6]

Times, with CUDA events on every rank (max over ranks, barrier between iterations), on a flat parameter space of the
size of Transformer-big:

* ``gather``        fsdp_gather of the whole space: every rank pulls (N-1)/N of the bf16 parameters from its peers;
* ``reduce``        reduce_unit over the whole space: every rank sums its 1/N piece over all N fp32 gradient buffers;
* ``update``        update_pieces: norm exchange, Adam(W) on the piece, peer stores of the refreshed bf16 parameters into
                    all N copies, clearing of the gradient buffer;
* ``allreduce_nccl`` the NCCL all-reduce of the same fp32 buffer, for comparison.

For each, the bytes that cross NVLink per rank and the fraction of the measured peer bandwidth (770 GB/s per direction)
that this corresponds to.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

NVLINK_GBS = 770.0


def timed(fn, iters, world):
    ms = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms.append(float(t))
    ms.sort()
    return ms[len(ms) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=209e6)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29519")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from nmtgminor_b200 import ops
    from nmtgminor_b200.options import default_options
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    from nmtgminor_b200.parallel.symmetric import FusedAllReduceAdam, SymmetricHeap
    from nmtgminor_b200.train.optim import Optim
    dev = torch.device("cuda", local)
    n = int(args.params) // (256 * world) * (256 * world)

    class Flat(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(n))

    model = Flat()
    heap = SymmetricHeap(dev)
    ptrs = {}

    def symm(name):
        def alloc(k, dt):
            t, p = heap.alloc(k, dt)
            ptrs[name] = p
            return t
        return alloc
    store = FlatParameterStore(model, dev, allocator={"grad": symm("grad"), "work": symm("work")}, pad_total_to=256 * world)
    opt = default_options(["-optim", "adam", "-learning_rate", "1e-4", "-update_method", "regular", "-weight_decay", "0.01",
                           "-max_grad_norm", "5"])
    optim = Optim(opt)
    optim.set_parameters(model.parameters(), store, allocate_state=False)
    fused = FusedAllReduceAdam(store, optim, heap, ptrs["grad"], ptrs["work"])
    optim.attach_distributed(fused)
    fused.reduce_ctas = int(os.environ.get("NMTG_REDUCE_CTAS", "296"))     # alone on the GPU: use all SMs
    store.grad.normal_(0, 0.01)
    u = fused.units[0]
    staging = torch.empty(u.piece * world, dtype=torch.bfloat16, device=dev)

    def gather():
        ops.ext().fsdp_gather(rank, ptrs["work"], staging, 0, u.piece, 0, u.piece * world, 296)

    def reduce():
        fused._done = set()
        fused(store.grad)

    def update():
        optim._step += 1
        optim.write_hyper(1.0)
        optim.launch_fused()

    def nccl():
        dist.all_reduce(store.grad)

    out = {"n_gpus": world, "params": n, "nvlink_gbs_per_direction": NVLINK_GBS}
    frac = (world - 1) / world
    for name, fn, nbytes in (("gather", gather, frac * n * 2), ("reduce", reduce, frac * n * 4), ("update", update, frac * n * 2),
                             ("allreduce_nccl", nccl, 2 * frac * n * 4)):
        for _ in range(3):
            fn()
        ms = timed(fn, args.iters, world)
        gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        out[name] = {"ms": ms, "nvlink_bytes_per_rank": nbytes, "gb_per_s": gbs, "fraction_of_link": gbs / NVLINK_GBS}
    torch.cuda.synchronize()
    out["kernel_status"] = ops.check_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

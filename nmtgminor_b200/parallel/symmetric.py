"""Symmetric (peer-mapped) device memory and the peer-memory optimiser step built on it.

``SymmetricHeap`` allocates buffers with plain ``cudaMalloc`` (so they can be exported), exchanges their CUDA
IPC handles through ``torch.distributed`` (any backend: the exchange is host-side bytes) and opens every
peer's handle; the result is, per buffer, one device pointer per rank.  This is the only use of the process
group on this path: bootstrap.

``FusedAllReduceAdam`` owns slice ``rank`` of the flat parameter space (fp32 master weights and Adam moments
exist only for that slice) and performs reduce-scatter + unscale + clip + Adam(W) + all-gather of the bf16
parameters + gradient clearing with the kernels of ``csrc/comm_p2p.cu`` - no NCCL call on the step.

``ShardedAdamReference`` is the same algorithm written with ``torch.distributed`` collectives (reduce-scatter,
all-gather of the norm partials, all-gather of parameters); it is what CPU / gloo tests run and what the
multi-GPU tests compare the kernels against.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from .. import ops

FLAG_INTS = 3 * 16
PARTIAL_FLOATS = 2 * 16


def slice_bounds(total: int, world: int, rank: int):
    assert total % (4 * world) == 0, "flat length must be a multiple of 4 * world size"
    n = total // world
    return rank * n, n


class SymmetricHeap:
    def __init__(self, device):
        self.device = torch.device(device)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self._keep = []       # owning tensors (cudaFree on release)
        self._opened = []     # peer pointers to close

    def alloc(self, numel: int, dtype: torch.dtype):
        """Returns (local tensor, [device pointer of this buffer on every rank])."""
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        raw = ops.ext().symm_alloc(int(nbytes), self.device.index)
        self._keep.append(raw)
        local = raw.view(dtype)[:numel]
        handle = ops.ext().ipc_get_handle(raw)
        handles: List[bytes] = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, handle)
        else:
            handles = [handle]
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(raw.data_ptr())
            else:
                p = ops.ext().ipc_open_handle(h, self.device.index)
                self._opened.append(p)
                ptrs.append(p)
        return local, ptrs

    def close(self):
        for p in self._opened:
            ops.ext().ipc_close_handle(p)
        self._opened = []
        self._keep = []


class FusedAllReduceAdam:
    """Peer-memory data-parallel step.  ``store.grad`` / ``store.work`` must come from ``heap``."""

    fused_optimizer = True

    def __init__(self, store, optim, heap: SymmetricHeap, grad_ptrs, work_ptrs):
        self.store, self.optim, self.heap = store, optim, heap
        self.rank, self.world = heap.rank, heap.world
        self.begin, self.length = slice_bounds(store.total, self.world, self.rank)
        dev = store.master.device
        flags, self.flag_ptrs = heap.alloc(FLAG_INTS, torch.int32)
        partials, self.partial_ptrs = heap.alloc(PARTIAL_FLOATS, torch.float32)
        self.flags, self.partials = flags, partials
        self.grad_ptrs, self.work_ptrs = grad_ptrs, work_ptrs
        self.reduced = torch.zeros(self.length, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.length, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.length, dtype=torch.float32, device=dev)
        self.sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.nonfinite = torch.zeros(1, dtype=torch.int32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.epoch = torch.ones(1, dtype=torch.int32, device=dev)
        if self.world > 1:
            dist.barrier()      # every rank has zeroed flags and opened every handle before the first step

    def __call__(self, flat_grad):   # the reduction happens inside ``launch`` together with the update
        return None

    def launch(self):
        s = self.store
        ops.ext().allreduce_adamw(self.rank, self.grad_ptrs, self.work_ptrs, self.flag_ptrs, self.partial_ptrs, self.reduced,
                                  self.sq, self.nonfinite, s.master[self.begin:self.begin + self.length], self.exp_avg,
                                  self.exp_avg_sq, self.optim.hyper, self.begin, self.length, s.total, self.epoch, self.norm)

    def gather_master(self):
        """Refresh the full fp32 master buffer on every rank from the owners' slices (before saving)."""
        if self.world > 1:
            mine = self.store.master[self.begin:self.begin + self.length].clone()
            dist.all_gather_into_tensor(self.store.master, mine)

    def state_dict(self):
        return {"exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(), "begin": self.begin, "length": self.length}


class ShardedAdamReference:
    """Collective-based statement of the same step (works on CPU with gloo and on GPU with NCCL)."""

    def __init__(self, total: int, device, beta1=0.9, beta2=0.997, eps=1e-9, weight_decay=0.0, max_grad_norm=0.0,
                 decoupled=True):
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.begin, self.length = slice_bounds(total, self.world, self.rank)
        self.m = torch.zeros(self.length, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.length, dtype=torch.float32, device=device)
        self.cfg = dict(beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                        decoupled=decoupled)
        self.t = 0

    def step(self, master_full: torch.Tensor, grad_full: torch.Tensor, lr: float, grad_scale: float = 1.0):
        from ..ops.reference import adamw_step
        self.t += 1
        if self.world > 1:
            chunks = list(grad_full.view(self.world, self.length).unbind(0))
            mine = torch.empty_like(chunks[0])
            if grad_full.is_cuda:
                dist.reduce_scatter(mine, chunks)
            else:   # gloo has no reduce_scatter: all-reduce then slice
                g = grad_full.clone()
                dist.all_reduce(g)
                mine = g[self.begin:self.begin + self.length].clone()
        else:
            mine = grad_full[self.begin:self.begin + self.length].clone()
        sq = (mine.double() ** 2).sum().reshape(1)
        if self.world > 1:
            dist.all_reduce(sq)
        norm = float(sq.sqrt()) * grad_scale
        coef = grad_scale
        mg = self.cfg["max_grad_norm"]
        if mg > 0 and norm > mg:
            coef *= mg / (norm + 1e-6)
        my_master = master_full[self.begin:self.begin + self.length]
        adamw_step(my_master, mine, self.m, self.v, lr=lr, beta1=self.cfg["beta1"], beta2=self.cfg["beta2"], eps=self.cfg["eps"],
                   weight_decay=self.cfg["weight_decay"], step=self.t, grad_scale=coef, max_grad_norm=0.0,
                   decoupled=self.cfg["decoupled"])
        if self.world > 1:
            dist.all_gather_into_tensor(master_full, my_master.clone()) if master_full.is_cuda else \
                dist.all_gather(list(master_full.view(self.world, self.length).unbind(0)), my_master.clone())
        grad_full.zero_()
        return norm

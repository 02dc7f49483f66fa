"""Symmetric (peer-mapped) device memory and the peer-memory optimiser step built on it.

``SymmetricHeap`` allocates buffers with plain ``cudaMalloc`` (so they can be exported), exchanges their CUDA
IPC handles through ``torch.distributed`` (any backend: the exchange is host-side bytes) and opens every
peer's handle; the result is, per buffer, one device pointer per rank.  This is the only use of the process
group on this path: bootstrap.

``FusedAllReduceAdam`` owns one piece of every layer of the flat parameter space (Adam moments exist only for
owned pieces) and performs per-layer reduce-scatter overlapped with the backward pass + unscale + clip + Adam(W)
+ all-gather of the bf16 parameters + gradient clearing with the kernels of ``csrc/comm_p2p.cu`` - no NCCL call
on the step.

``ShardedAdamReference`` is the same algorithm written with ``torch.distributed`` collectives (reduce-scatter,
all-gather of the norm partials, all-gather of parameters); it is what CPU / gloo tests run and what the
multi-GPU tests compare the kernels against.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from .. import ops
from .sharded import FLAG_INTS, PARTIAL_FLOATS, UnitShardedStep, plan_units  # noqa: F401  (re-exported)


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


class FusedAllReduceAdam(UnitShardedStep):
    """Peer-memory data-parallel step.  ``store.grad`` / ``store.work`` must come from ``heap``.

    Every rank keeps full fp32 gradients, a full bf16 parameter copy and the full fp32 master buffer (of which only
    the owned pieces are current between checkpoints); Adam moments exist only for the owned pieces.  Per step:
    per-layer ``reduce_unit`` launches overlapped with the backward pass, then one ``update_pieces`` launch whose
    peer stores refresh every rank's bf16 copy (see ``sharded.UnitShardedStep``)."""

    mode = 0

    def __init__(self, store, optim, heap: SymmetricHeap, grad_ptrs, work_ptrs, model=None, overlap: bool = True):
        units = plan_units(model, store, heap.world) if model is not None else plan_units(torch.nn.Module(), store, heap.world)
        self._setup(model, store, optim, heap, grad_ptrs, work_ptrs, units, overlap=overlap)
        if self.world > 1:
            dist.barrier()      # every rank has zeroed flags and opened every handle before the first step

    def gather_master(self):
        """Refresh the full fp32 master buffer on every rank from the owners' pieces (before saving)."""
        if self.world <= 1:
            return
        mine = torch.zeros(self.shard_len, dtype=torch.float32, device=self.device)
        for (so, p0, n), u in zip(self.pieces, self.units):
            full = max(0, min(u.piece, u.end - p0))
            if full > 0:
                mine[so:so + full].copy_(self.store.master[p0:p0 + full])
        everyone = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(everyone, mine)
        for r, shard in enumerate(everyone):
            if r != self.rank:
                self._shard_to_flat(shard, self.store.master, r)


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

"""
Peer-memory ("fused") communication backend for the FSDP shard group.

The bf16 compute copy of the parameters and the fp32 gradient accumulator are allocated in symmetric memory
(``torch.distributed._symmetric_memory``: every rank of the group maps every other rank's buffer over NVLink), which
lets our kernels fuse the FSDP collectives into the GEMMs instead of calling NCCL:

* **all-gather -> GEMM**: a weight is never gathered by a separate collective.  The first GEMM that needs it gets a
  table of the peers' shard addresses; its copy warps stream the remote shards into the local staging buffer while
  its tensor-core warps already work on the local shard, and tiles of a remote shard wait on per-block arrival
  counters (``csrc/gemm.cu``).  The embedding gather reads rows straight from the owner GPU.
* **GEMM -> reduce-scatter**: the weight-gradient GEMM's epilogue adds each row block into the owner GPU's fp32
  accumulator with ``red.global.add`` (scaled by 1 / (ranks x micro-batches)), so there is no reduce-scatter at all.

Only plain loads / stores / reductions touch peer memory; TMA descriptors always point at local memory.  Two
stream-ordered barriers per optimizer step (before it: every peer's reductions have landed and nobody still reads
our weights; after it: every peer's new weights are visible and its accumulator is cleared) are the only
synchronisation between ranks.
"""

from __future__ import annotations

import logging
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K

__all__ = ["SymmContext", "symm_available"]

log = logging.getLogger(__name__)


def symm_available(device: torch.device) -> bool:
    if device.type != "cuda" or not dist.is_available() or not dist.is_initialized():
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return dist.get_backend() == "nccl"


class SymmContext:
    def __init__(self, store, numel: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.store = store
        group = store.mesh.shard
        self.group = group
        self.R = group.size
        self.rank = group.rank
        dev = store.device
        self.shadow = symm_mem.empty(numel, dtype=store.compute_dtype, device=dev)
        self.grad = symm_mem.empty(numel, dtype=torch.float32, device=dev)
        self.shadow.zero_()
        self.grad.zero_()
        self._h_shadow = symm_mem.rendezvous(self.shadow, group.pg)
        self._h_grad = symm_mem.rendezvous(self.grad, group.pg)
        self.shadow_ptrs: List[int] = [int(p) for p in self._h_shadow.buffer_ptrs]
        self.grad_ptrs: List[int] = [int(p) for p in self._h_grad.buffer_ptrs]
        self.flags = torch.zeros(self.R * 4096, dtype=torch.int32, device=dev)
        self._tables: Dict[tuple, torch.Tensor] = {}
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        self.multicast_ptr = int(getattr(self._h_grad, "multicast_ptr", 0) or 0)
        log.info("Peer-memory backend on: %d ranks, %.1f MiB bf16 weights + %.1f MiB fp32 gradients mapped per rank",
                 self.R, numel * 2 / 2**20, numel * 4 / 2**20)

    def _table(self, kind: str, handle, base_ptrs: List[int], elem_size: int) -> torch.Tensor:
        key = (kind, handle.name)
        t = self._tables.get(key)
        if t is None:
            off = handle.meta.offset * elem_size
            t = K.pointer_table([p + off for p in base_ptrs], self.store.device)
            self._tables[key] = t
        return t

    def grad_pointer_table(self, handle) -> torch.Tensor:
        """Device array of the R addresses where the row shards of ``handle``'s gradient live (one per GPU)."""
        return self._table("grad", handle, self.grad_ptrs, 4)

    def shadow_pointer_table(self, handle) -> torch.Tensor:
        return self._table("shadow", handle, self.shadow_ptrs, self.shadow.element_size())

    def unit_pointer_table(self, unit) -> torch.Tensor:
        """Device array of the R addresses of ``unit``'s slice of the bf16 weights (one per GPU)."""
        key = ("unit", unit.name)
        t = self._tables.get(key)
        if t is None:
            off = unit.offset * self.shadow.element_size()
            t = K.pointer_table([p + off for p in self.shadow_ptrs], self.store.device)
            self._tables[key] = t
        return t

    def sync_peers(self) -> None:
        """Stream-ordered barrier over the shard group (a one-element NCCL all-reduce)."""
        dist.all_reduce(self._token, group=self.group.pg)

"""
Sharded parameter storage and the FSDP engine.

Every parameter is split on dim 0 over the FSDP shard group (after an optional tensor-parallel split of dim 0 or 1),
exactly the placement the reference requests from GSPMD (``olmax/distributed/parallel.py:309-334``,
``olmax/nn/linear.py:46-54``).  What differs is the memory layout, which is chosen for the kernels:

* Per rank there is ONE flat fp32 master buffer, ONE flat fp32 gradient accumulator and ONE flat compute-dtype
  ("shadow", bf16) buffer; a parameter's local shard is a view into them.  The optimizer runs as a few launches over
  the flat buffers, the HSDP/DDP all-reduce is one collective over the flat gradient, and the bf16 shadow is written
  by the optimizer so no per-micro-batch cast is needed.
* Parameters are grouped into *units* (embedding, each transformer layer, final norm + head).  A unit's shards are
  contiguous, so ONE all-gather of the shadow slice brings in the whole unit as a rank-major ``[R, unit_numel]``
  buffer.  GEMM kernels read a weight straight out of that buffer as ``R`` row blocks ``unit_numel`` apart, so no
  re-layout copy is made; weight-gradient GEMMs write the mirrored ``[R, unit_numel]`` fp32 buffer that a single
  reduce-scatter turns into the local gradient shard.
* Gathers are prefetched one unit ahead (forward and backward) and reduce-scatters are left in flight until the end
  of the backward pass.

On a shard group of one (single GPU, DDP) all of this collapses to views of the local buffers.
"""

from __future__ import annotations

import fnmatch
import logging
import math
import os
import zlib
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..exceptions import OLMaxConfigurationError
from ..ops import kernels as K
from ..utils.tree import fold_in
from . import collectives as coll
from .mesh import DeviceMesh

__all__ = ["ParamMeta", "ParamHandle", "FSDPUnit", "ParamStore"]

log = logging.getLogger(__name__)


@dataclass
class ParamMeta:
    name: str
    shape: Tuple[int, ...]          # logical (unsharded) shape
    unit: str
    tp_dim: Optional[int] = None    # dim split over the TP axis (None: replicated over TP)
    decay: bool = True
    init: str = "trunc_normal"      # trunc_normal | normal | ones | zeros
    init_std: float = 0.02
    # filled by ParamStore.finalize
    tp_shape: Tuple[int, ...] = ()
    local_shape: Tuple[int, ...] = ()
    offset: int = 0                 # element offset of the local shard in the flat buffers
    unit_offset: int = 0            # element offset inside the unit
    numel_local: int = 0


class ParamHandle:
    """What a module holds instead of an ``nn.Parameter``: access to the shard, the gathered weight and the gradient."""

    def __init__(self, store: "ParamStore", meta: ParamMeta):
        self.store = store
        self.meta = meta
        self.unit: Optional["FSDPUnit"] = None

    # ---- local views -------------------------------------------------------------------------------------------
    def _view(self, flat: torch.Tensor) -> torch.Tensor:
        m = self.meta
        return flat[m.offset : m.offset + m.numel_local].view(m.local_shape)

    @property
    def local_master(self) -> torch.Tensor:
        return self._view(self.store.master)

    @property
    def local_grad(self) -> torch.Tensor:
        return self._view(self.store.grad)

    @property
    def local_shadow(self) -> torch.Tensor:
        return self._view(self.store.shadow)

    @property
    def name(self) -> str:
        return self.meta.name

    @property
    def shard_count(self) -> int:
        return self.store.mesh.shard.size

    @property
    def rows_local(self) -> int:
        return self.meta.local_shape[0]

    @property
    def tp_shape(self) -> Tuple[int, ...]:
        return self.meta.tp_shape

    # ---- gathered access ---------------------------------------------------------------------------------------
    def pieces(self) -> Tuple[torch.Tensor, int]:
        """(rank-0 piece view, element stride between consecutive ranks' pieces) of the gathered weight."""
        assert self.unit is not None
        buf = self.unit.gathered()
        m = self.meta
        first = buf[0, m.unit_offset : m.unit_offset + m.numel_local].view(m.local_shape)
        return first, buf.stride(0)

    def full(self) -> torch.Tensor:
        """The TP-local weight in compute dtype, assembled from the gathered unit (a view when the group is 1)."""
        assert self.unit is not None
        R = self.shard_count
        m = self.meta
        buf = self.unit.gathered()
        if R == 1:
            return buf[0, m.unit_offset : m.unit_offset + m.numel_local].view(m.local_shape)
        cached = self.unit._full_cache.get(m.name)
        if cached is None:
            if m.name in self.unit._ag_pending:
                # small tensors (norm weights, biases) read through full(): fetch the peers' shards with our own
                # plain-load kernel
                K.gather_shards(self.store.symm.shadow_pointer_table(self), buf[0, m.unit_offset:], buf.stride(0),
                                m.numel_local, R, self.store.mesh.shard.rank)
                self.unit._ag_pending.discard(m.name)
            cached = buf[:, m.unit_offset : m.unit_offset + m.numel_local].reshape(m.tp_shape)
            self.unit._full_cache[m.name] = cached
        return cached

    def take_ag(self):
        """(peer pointer table, flags, rank) when this weight's remote shards still have to be fetched into the
        gathered buffer by the next GEMM, else None; marks the weight as fetched."""
        if self.unit is None or self.name not in self.unit._ag_pending:
            return None
        self.unit._ag_pending.discard(self.name)
        symm = self.store.symm
        return symm.shadow_pointer_table(self), symm.flags, self.store.mesh.shard.rank

    # ---- gradients ---------------------------------------------------------------------------------------------
    def grad_pieces(self) -> Tuple[torch.Tensor, int, float]:
        """
        (rank-0 piece view of the fp32 destination for this weight's full gradient, element stride between ranks'
        pieces, scale to apply when accumulating).  With a shard group of one the destination is the local gradient
        accumulator itself and the scale is the final 1/(dp*k); otherwise it is the unit's full-gradient buffer
        (scale 1; the scale is applied after the reduce-scatter).
        """
        assert self.unit is not None
        m = self.meta
        if self.shard_count == 1:
            return self.local_grad, 0, self.store.grad_scale
        buf = self.unit.full_grad()
        first = buf[0, m.unit_offset : m.unit_offset + m.numel_local].view(m.local_shape)
        return first, buf.stride(0), 1.0

    def add_grad(self, g_full: torch.Tensor) -> None:
        """Accumulate a full (TP-local) gradient computed with ordinary tensor math (CPU path, small params)."""
        m = self.meta
        if self.store.symm_rs is not None and self.shard_count > 1:
            K.scatter_add_shards(g_full.reshape(-1).float().contiguous(), self.store.symm.grad_pointer_table(self),
                                 m.numel_local, self.shard_count, self.store.grad_scale)
            return
        first, stride, scale = self.grad_pieces()
        if self.shard_count == 1:
            first.add_(g_full.reshape(m.local_shape).to(first.dtype), alpha=scale)
            return
        buf = self.unit.full_grad()
        dst = buf[:, m.unit_offset : m.unit_offset + m.numel_local]
        dst.add_(g_full.reshape(self.shard_count, m.numel_local).to(dst.dtype))


class FSDPUnit:
    """A group of parameters gathered / reduced together."""

    def __init__(self, store: "ParamStore", name: str, index: int):
        self.store = store
        self.name = name
        self.index = index
        self.params: List[ParamHandle] = []
        self.offset = 0
        self.numel_local = 0
        self._gathered: Optional[torch.Tensor] = None
        self._gather_work = None
        self._full_grad: Optional[torch.Tensor] = None
        self._full_cache: Dict[str, torch.Tensor] = {}
        self._ag_pending: set = set()
        self._staged: set = set()   # parameters whose weight gradient sits in the peers' staging slots
        self._pf_cursor = 0
        self.numel_full_2d = 1
        self.lazy = False  # True: only gather when a consumer actually asks for the gathered buffer

    # ---- gather ------------------------------------------------------------------------------------------------
    def start_gather(self, force: bool = False) -> None:
        if self._gathered is not None or (self.lazy and not force):
            return
        st = self.store
        R = st.mesh.shard.size
        local = st.shadow[self.offset : self.offset + self.numel_local]
        if R == 1:
            self._gathered = local.view(1, -1)
            return
        buf = st._take_buffer("gather", R * self.numel_local, st.compute_dtype).view(R, self.numel_local)
        if st.symm_ag is not None:
            # peer-memory backend: only the local slot is filled here; every weight's remote slots are fetched by the
            # first GEMM that uses it (all-gather fused into the GEMM)
            buf[st.mesh.shard.rank].copy_(local)
            self._ag_pending = {h.name for h in self.params}
            self._pf_cursor = 0
            self._gathered = buf
            return
        self._gather_work = coll.all_gather_into(buf, local, st.mesh.shard, async_op=True)
        self._gathered = buf
        st.stats["all_gather_bytes"] += (R - 1) * self.numel_local * local.element_size()

    def gathered(self) -> torch.Tensor:
        if self._gathered is None:
            self.start_gather(force=True)
        if self._gather_work is not None:
            self._gather_work.wait()
            self._gather_work = None
        return self._gathered  # type: ignore[return-value]

    def release(self) -> None:
        if self._gather_work is not None:
            self._gather_work.wait()
            self._gather_work = None
        if self._gathered is not None and self.store.mesh.shard.size > 1:
            self.store._give_buffer("gather", self._gathered)
        self._gathered = None
        self._ag_pending = set()
        self._pf_cursor = 0
        if self.store._pf_unit is self:
            self.store._pf_unit = None
        self._full_cache.clear()

    # ---- gradients ---------------------------------------------------------------------------------------------
    def full_grad(self) -> torch.Tensor:
        if self._full_grad is None:
            st = self.store
            R = st.mesh.shard.size
            buf = st._take_buffer("grad", R * self.numel_local, st.grad_comm_dtype).view(R, self.numel_local)
            buf.zero_()
            self._full_grad = buf
        return self._full_grad

    def reduce_grads(self) -> None:
        """Reduce-scatter this unit's full gradient into the local accumulator (asynchronously on the GPU)."""
        st = self.store
        if self._staged:
            # peer-memory backend: every rank's weight-gradient GEMMs have stored their contributions into the owners'
            # staging slots; after a barrier each owner folds its slots into its accumulator
            names, self._staged = self._staged, set()
            st.symm.rs_unit_done(self, names)
            st.stats["reduce_scatter_bytes"] += (st.mesh.shard.size - 1) * self.numel_local * 4
        if self._full_grad is None:
            return
        R = st.mesh.shard.size
        buf = self._full_grad
        self._full_grad = None
        out = st._take_buffer("rs_out", self.numel_local, st.grad_comm_dtype)
        if buf.is_cuda:
            work = dist.reduce_scatter_tensor(out, buf.view(-1), group=st.mesh.shard.pg, async_op=True)
        else:
            coll.reduce_scatter_into(out, buf.view(-1), st.mesh.shard, predivide=False)
            work = None
        st.stats["reduce_scatter_bytes"] += (R - 1) * self.numel_local * buf.element_size()
        st._pending_reduce.append((self, work, buf, out))
        # keep one reduce-scatter in flight: fold the older ones now so that their full-size buffers return to the pool
        # (otherwise a whole model's worth of un-reduced fp32 gradients is alive at the end of the backward pass)
        while len(st._pending_reduce) > 1:
            st._fold_pending(st._pending_reduce.pop(0))


class ParamStore:
    def __init__(
        self,
        mesh: DeviceMesh,
        param_dtype: torch.dtype = torch.float32,
        compute_dtype: torch.dtype = torch.bfloat16,
        device: Optional[torch.device] = None,
        reshard_after_forward: bool = True,
        comm_backend: Optional[str] = None,
    ):
        self.mesh = mesh
        self.comm_backend = comm_backend or os.environ.get("OLMAX_B200_COMM_BACKEND", "auto")
        self.param_dtype = param_dtype
        self.compute_dtype = compute_dtype
        self.grad_comm_dtype = torch.float32
        self.device = device if device is not None else mesh.device
        self.reshard_after_forward = reshard_after_forward
        self.metas: List[ParamMeta] = []
        self.handles: Dict[str, ParamHandle] = {}
        self.units: List[FSDPUnit] = []
        self._unit_by_name: Dict[str, FSDPUnit] = {}
        self.master: torch.Tensor = torch.empty(0)
        self.grad: torch.Tensor = torch.empty(0)
        self.shadow: torch.Tensor = torch.empty(0)
        self.numel_local = 0
        self.grad_scale = 1.0
        self._pool: Dict[str, List[torch.Tensor]] = {}
        self._pending_reduce: List = []
        self.stats: Dict[str, int] = {"all_gather_bytes": 0, "reduce_scatter_bytes": 0, "all_reduce_bytes": 0}
        self._finalized = False
        self.symm = None  # symmetric-memory context when the fused backend is active
        self._pf_unit: Optional[FSDPUnit] = None
        self._in_backward = False
        self.symm_ag = None  # ... used for the all-gather side (weights fetched inside the GEMMs)
        self.symm_rs = None  # ... used for the reduce-scatter side (gradients added into the owners' shards)
        self.tp_symm = None  # peer-memory context of the tensor-parallel group (collectives fused into the GEMMs)

    # ------------------------------------------------------------------ registration
    def register(
        self,
        name: str,
        shape: Sequence[int],
        unit: str,
        tp_dim: Optional[int] = None,
        decay: bool = True,
        init: str = "trunc_normal",
        init_std: float = 0.02,
    ) -> ParamHandle:
        if self._finalized:
            raise RuntimeError("ParamStore is finalized")
        if name in self.handles:
            raise OLMaxConfigurationError(f"duplicate parameter name '{name}'")
        meta = ParamMeta(name=name, shape=tuple(int(s) for s in shape), unit=unit, tp_dim=tp_dim, decay=decay,
                         init=init, init_std=init_std)
        tp = self.mesh.tp.size
        tp_shape = list(meta.shape)
        if tp_dim is not None and tp > 1:
            if tp_shape[tp_dim] % tp != 0:
                raise OLMaxConfigurationError(f"{name}: dim {tp_dim} ({tp_shape[tp_dim]}) not divisible by tp={tp}")
            tp_shape[tp_dim] //= tp
        R = self.mesh.shard.size
        if tp_shape[0] % R != 0:
            raise OLMaxConfigurationError(
                f"{name}: dim 0 ({tp_shape[0]}) is not divisible by the FSDP shard degree {R}; pad it (for a "
                f"vocabulary use a size that is a multiple of the shard degree)"
            )
        meta.tp_shape = tuple(tp_shape)
        meta.local_shape = (tp_shape[0] // R,) + tuple(tp_shape[1:])
        meta.numel_local = int(math.prod(meta.local_shape))
        handle = ParamHandle(self, meta)
        if unit not in self._unit_by_name:
            u = FSDPUnit(self, unit, len(self.units))
            self.units.append(u)
            self._unit_by_name[unit] = u
        u = self._unit_by_name[unit]
        u.params.append(handle)
        handle.unit = u
        self.metas.append(meta)
        self.handles[name] = handle
        return handle

    def finalize(self, seed: int = 0, init: bool = True) -> None:
        """Lay out the flat buffers (units in registration order), allocate and initialise them."""
        if self._finalized:
            return
        off = 0
        align = 64  # elements: keeps every shard 128-byte aligned in bf16 (TMA needs 16)
        for u in self.units:
            u.offset = off
            uoff = 0
            for h in u.params:
                h.meta.unit_offset = uoff
                h.meta.offset = off + uoff
                uoff += (h.meta.numel_local + align - 1) // align * align
            u.numel_local = uoff
            u.numel_full_2d = max(1, sum(int(math.prod(h.meta.tp_shape)) for h in u.params if len(h.meta.shape) == 2))
            off += uoff
        self.numel_local = off
        self.validate_layout()
        dev = self.device
        self.master = torch.zeros(off, dtype=self.param_dtype, device=dev)
        use_symm = False
        if (self.comm_backend in ("auto", "fused") and self.compute_dtype != self.param_dtype
                and (self.mesh.shard.size > 1 or self.mesh.replicate.size > 1)):
            from .symm import SymmContext, symm_available

            use_symm = symm_available(dev)
            if self.comm_backend == "fused" and not use_symm:
                raise OLMaxConfigurationError("comm_backend='fused' needs CUDA, NCCL and torch symmetric memory")
        if use_symm:
            self.symm = SymmContext(self, off)
            self.grad = self.symm.grad
            self.shadow = self.symm.shadow
            # experiment knobs: fall back to the NCCL collective for one direction while keeping the other fused
            sharded = self.mesh.shard.size > 1
            self.symm_ag = self.symm if (sharded and os.environ.get("OLMAX_B200_FUSED_AG", "1") == "1") else None
            self.symm_rs = self.symm if (sharded and os.environ.get("OLMAX_B200_FUSED_RS", "1") == "1") else None
        else:
            self.grad = torch.zeros(off, dtype=torch.float32, device=dev)
            if self.compute_dtype == self.param_dtype:
                self.shadow = self.master
            else:
                self.shadow = self._alloc_shadow(off)
        if (self.mesh.tp.size > 1 and dev.type == "cuda" and self.comm_backend in ("auto", "fused")
                and self.compute_dtype == torch.bfloat16 and os.environ.get("OLMAX_B200_FUSED_TP", "1") == "1"):
            from .symm import TPSymmContext, symm_available

            if symm_available(dev):
                self.tp_symm = TPSymmContext(self.mesh, dev)
            elif self.comm_backend == "fused":
                raise OLMaxConfigurationError("comm_backend='fused' needs CUDA, NCCL and torch symmetric memory")
        self._finalized = True
        if init:
            self.init_parameters(seed)

    def validate_layout(self) -> None:
        """Host-side check of the flat layout the kernels rely on: units tile the buffer in order, parameter slices lie
        inside their unit without overlapping, every slice starts on a 64-element boundary (128 bytes in bf16: TMA
        descriptors, 16-byte vector accesses and the line-coalesced peer stores all assume it) and every 2-D parameter's
        rows are a multiple of 8 elements long.  Raises ``OLMaxConfigurationError`` with the offending parameter."""
        end_prev_unit = 0
        for u in self.units:
            if u.offset != end_prev_unit:
                raise OLMaxConfigurationError(f"unit {u.name} starts at {u.offset}, expected {end_prev_unit}")
            end_prev = 0
            for h in u.params:
                m = h.meta
                if m.unit_offset % 64 or m.offset != u.offset + m.unit_offset:
                    raise OLMaxConfigurationError(f"{m.name}: slice offset {m.offset} (unit offset {m.unit_offset}) is misplaced")
                if m.unit_offset < end_prev:
                    raise OLMaxConfigurationError(f"{m.name}: slice overlaps the previous parameter of unit {u.name}")
                if m.numel_local != int(math.prod(m.local_shape)) or m.numel_local <= 0:
                    raise OLMaxConfigurationError(f"{m.name}: local shape {m.local_shape} does not match {m.numel_local} elements")
                if len(m.local_shape) == 2 and m.local_shape[1] % 8 and self.device.type == "cuda":
                    raise OLMaxConfigurationError(f"{m.name}: rows of {m.local_shape[1]} elements are not a multiple of 8 "
                                                  f"(16 bytes), which the TMA descriptors of the GEMM need")
                end_prev = m.unit_offset + m.numel_local
            if end_prev > u.numel_local:
                raise OLMaxConfigurationError(f"unit {u.name}: parameters extend past the unit ({end_prev} > {u.numel_local})")
            end_prev_unit = u.offset + u.numel_local
        if end_prev_unit != self.numel_local:
            raise OLMaxConfigurationError(f"flat buffer has {self.numel_local} elements, units cover {end_prev_unit}")

    def _alloc_shadow(self, numel: int) -> torch.Tensor:
        return torch.zeros(numel, dtype=self.compute_dtype, device=self.device)

    # ------------------------------------------------------------------ init
    def _init_full(self, meta: ParamMeta, seed: int) -> torch.Tensor:
        """The full logical tensor for ``meta`` from a stream that depends only on (seed, name)."""
        dev = self.device
        if meta.init == "ones":
            return torch.ones(meta.shape, dtype=torch.float32, device=dev)
        if meta.init == "zeros":
            return torch.zeros(meta.shape, dtype=torch.float32, device=dev)
        gen = torch.Generator(device=dev)
        gen.manual_seed(fold_in(seed, zlib.crc32(meta.name.encode())))
        t = torch.empty(meta.shape, dtype=torch.float32, device=dev)
        if meta.init == "trunc_normal":
            # std * TruncNormal(-3, 3): the truncated variate is not re-normalised (``olmax/nn/init.py:10-29``)
            torch.nn.init.trunc_normal_(t, mean=0.0, std=meta.init_std, a=-3 * meta.init_std, b=3 * meta.init_std,
                                        generator=gen)
        elif meta.init == "normal":
            t.normal_(0.0, meta.init_std, generator=gen)
        else:
            raise OLMaxConfigurationError(f"unknown init '{meta.init}' for {meta.name}")
        return t

    def local_slice_of(self, meta: ParamMeta, full: torch.Tensor) -> torch.Tensor:
        """This rank's shard of a full logical tensor."""
        t = full
        tp = self.mesh.tp
        if meta.tp_dim is not None and tp.size > 1:
            t = t.chunk(tp.size, dim=meta.tp_dim)[tp.rank]
        sh = self.mesh.shard
        if sh.size > 1:
            t = t.chunk(sh.size, dim=0)[sh.rank]
        return t

    def init_parameters(self, seed: int = 0) -> None:
        for meta in self.metas:
            full = self._init_full(meta, seed)
            self.handles[meta.name].local_master.copy_(self.local_slice_of(meta, full).to(self.param_dtype))
            del full
        self.sync_shadow()

    def sync_shadow(self) -> None:
        """Refresh the compute-dtype copy from the master weights (the fused optimizer does this by itself)."""
        if self.shadow is not self.master:
            self.shadow.copy_(self.master)
        self.invalidate_gathered()
        self.sync_peers()

    # ------------------------------------------------------------------ buffer pool
    def _take_buffer(self, kind: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        free = self._pool.setdefault(kind, [])
        best = None
        for i, b in enumerate(free):
            if b.dtype == dtype and b.numel() >= numel and (best is None or b.numel() < free[best].numel()):
                best = i
        if best is not None:
            return free.pop(best)[:numel]
        return torch.empty(numel, dtype=dtype, device=self.device)

    def _give_buffer(self, kind: str, buf: torch.Tensor) -> None:
        base = buf.view(-1)
        root = base._base if base._base is not None else base
        self._pool.setdefault(kind, []).append(root.view(-1))

    # ------------------------------------------------------------------ step protocol
    def set_grad_scale(self, scale: float) -> None:
        """Factor applied to every gradient contribution: 1 / (ranks sharing one loss mean * micro-batches)."""
        self.grad_scale = float(scale)

    def unit(self, name: str) -> FSDPUnit:
        return self._unit_by_name[name]

    def prefetch(self, unit_index: int) -> None:
        """Start bringing in the weights of a unit that will be needed soon.  NCCL backend: launch its all-gather.
        Peer-memory backend: allocate its staging buffer and make it the target that subsequent GEMM launches stream
        remote shards into (see :meth:`prefetch_slice`)."""
        if not (0 <= unit_index < len(self.units)):
            return
        u = self.units[unit_index]
        u.start_gather()
        if self.symm_ag is not None and self.mesh.shard.size > 1:
            self._pf_unit = u if u._pf_cursor < u.numel_local * self.shadow.element_size() else None

    def prefetch_slice(self, weight_numel: int):
        """Arguments that let one GEMM launch carry part of the prefetch target's all-gather: the launch copies a byte
        range of every remote shard's slice of that unit, sized in proportion to the GEMM's own weight so that the copy
        takes about as long as the math.  Parameters whose bytes are covered stop being pending."""
        u = self._pf_unit
        if u is None or u._gathered is None or self.symm_ag is None:
            return None
        es = self.shadow.element_size()
        total = u.numel_local * es
        if u._pf_cursor >= total:
            self._pf_unit = None
            return None
        passes = 2.0 if self._in_backward else 1.0
        frac = 1.25 * weight_numel / max(1.0, u.numel_full_2d * passes)
        nbytes = min(total - u._pf_cursor, (int(total * frac) + 15) // 16 * 16)
        if nbytes <= 0:
            return None
        off = u._pf_cursor
        u._pf_cursor += nbytes
        for h in u.params:
            if (h.meta.unit_offset + h.meta.numel_local) * es <= u._pf_cursor:
                u._ag_pending.discard(h.name)
        buf = u._gathered
        return (self.symm_ag.unit_pointer_table(u), buf.data_ptr(), buf.stride(0) * es, off, nbytes,
                self.mesh.shard.size, self.mesh.shard.rank)

    def reduce_unit_now(self, unit: FSDPUnit) -> None:
        """Reduce-scatter ``unit``'s weight gradients and fold them into the accumulator without deferring the fold
        (used for gradients produced outside the backward order of the units)."""
        unit.reduce_grads()
        if self.symm_rs is not None:
            self.symm_rs.rs_flush()

    def invalidate_gathered(self) -> None:
        for u in self.units:
            u.release()

    def finish_backward(self) -> None:
        """Reduce any unit whose gradient is still un-reduced (embedding: its backward runs last), wait for the
        in-flight reduce-scatters, fold them into the fp32 accumulators and drop gathered weights."""
        self._in_backward = False
        for u in self.units:
            if u._full_grad is not None or u._staged:
                u.reduce_grads()
        if self.symm_rs is not None:
            self.symm_rs.rs_flush()
        if self.reshard_after_forward and self.mesh.shard.size > 1:
            for u in self.units:
                u.release()
        while self._pending_reduce:
            self._fold_pending(self._pending_reduce.pop(0))

    def _fold_pending(self, item) -> None:
        unit, work, buf, out = item
        if work is not None:
            work.wait()   # stream-ordered: the compute stream waits for the collective, the host does not
        self.grad[unit.offset : unit.offset + unit.numel_local].add_(out, alpha=self.grad_scale)
        self._give_buffer("grad", buf)
        self._give_buffer("rs_out", out)

    def reduce_replicated_grads(self) -> None:
        """
        Once per optimizer step (after the LAST micro-batch): sum the accumulated gradient over the replicate axes
        (HSDP / DDP) and, for parameters replicated over the TP axis, over that axis too.  The reference performs the
        cross-replica all-reduce after every micro-batch; doing it once is mathematically identical because the
        accumulator is linear in the micro-batch gradients.
        """
        self.sync_peers()
        rep = self.mesh.replicate
        if rep.size > 1 and self.symm is not None and os.environ.get("OLMAX_B200_FUSED_AR", "1") == "1":
            self.stats["all_reduce_bytes"] += self.symm.all_reduce_replicas()
            self.sync_peers()
        elif rep.size > 1:
            coll.all_reduce(self.grad, rep)
            self.stats["all_reduce_bytes"] += 2 * (rep.size - 1) * self.grad.numel() * 4 // rep.size
        tp = self.mesh.tp
        if tp.size > 1:
            for run_start, run_end in self._runs(lambda m: m.tp_dim is None):
                coll.all_reduce(self.grad[run_start:run_end], tp)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def sync_peers(self) -> None:
        """With the peer-memory backend: stream-ordered barrier over the shard group.  It separates the phases in
        which ranks write into each other's gradient shards / read each other's weights from the optimizer step."""
        if self.symm is not None:
            self.symm.sync_peers()

    def _runs(self, pred: Callable[[ParamMeta], bool]) -> List[Tuple[int, int]]:
        """Maximal contiguous [start, end) ranges of the flat buffer whose parameters satisfy ``pred``."""
        runs: List[Tuple[int, int]] = []
        metas = sorted(self.metas, key=lambda m: m.offset)
        for i, m in enumerate(metas):
            if not pred(m):
                continue
            end = metas[i + 1].offset if i + 1 < len(metas) else self.numel_local
            if runs and runs[-1][1] == m.offset:
                runs[-1] = (runs[-1][0], end)
            else:
                runs.append((m.offset, end))
        return runs

    def decay_runs(self) -> Tuple[List[Tuple[int, int]], List[Tuple[int, int]]]:
        return self._runs(lambda m: m.decay), self._runs(lambda m: not m.decay)

    def apply_decay_mask(self, no_decay_patterns: Optional[Iterable[str]]) -> None:
        """Mark parameters whose dotted name matches one of the glob patterns as exempt from weight decay
        (``olmax/optim/config.py:93-122``)."""
        pats = list(no_decay_patterns or [])
        for m in self.metas:
            m.decay = not any(fnmatch.fnmatch(m.name, p) for p in pats)

    # ------------------------------------------------------------------ logical (unsharded) access
    def _gather_logical(self, meta: ParamMeta, flat: torch.Tensor) -> torch.Tensor:
        local = flat[meta.offset : meta.offset + meta.numel_local].view(meta.local_shape)
        t = coll.all_gather(local.contiguous(), self.mesh.shard, dim=0)
        if meta.tp_dim is not None and self.mesh.tp.size > 1:
            t = coll.all_gather(t.contiguous(), self.mesh.tp, dim=meta.tp_dim)
        return t

    def full_parameter(self, name: str) -> torch.Tensor:
        """The unsharded fp32 master value (collective over the shard and TP groups)."""
        return self._gather_logical(self.handles[name].meta, self.master)

    def full_gradient(self, name: str) -> torch.Tensor:
        return self._gather_logical(self.handles[name].meta, self.grad)

    def full_tensor_like(self, name: str, flat: torch.Tensor) -> torch.Tensor:
        """Unsharded view of any flat buffer laid out like the master (optimizer moments)."""
        return self._gather_logical(self.handles[name].meta, flat)

    def load_full(self, name: str, full: torch.Tensor, flat: Optional[torch.Tensor] = None) -> None:
        """Write this rank's shard of an unsharded tensor into ``flat`` (default: master)."""
        meta = self.handles[name].meta
        if tuple(full.shape) != meta.shape:
            raise OLMaxConfigurationError(f"{name}: expected shape {meta.shape}, got {tuple(full.shape)}")
        target = self.master if flat is None else flat
        dst = target[meta.offset : meta.offset + meta.numel_local].view(meta.local_shape)
        dst.copy_(self.local_slice_of(meta, full.to(self.device)).to(dst.dtype))

    def named_parameters(self) -> List[Tuple[str, ParamHandle]]:
        return [(m.name, self.handles[m.name]) for m in self.metas]

    def num_parameters(self) -> int:
        return sum(int(math.prod(m.shape)) for m in self.metas)

    def global_grad_sumsq(self) -> torch.Tensor:
        """Sum of squares of the full gradient (fp32 scalar tensor, identical on all ranks).  TP-replicated
        parameters are counted once."""
        tp = self.mesh.tp
        if self.grad.is_cuda:
            # no temporaries: the reduction kernel accumulates straight into two fp64 scalars
            acc = torch.zeros(2, dtype=torch.float64, device=self.device)
            if tp.size > 1:
                for s, e in self._runs(lambda m: m.tp_dim is not None):
                    K.sumsq(self.grad[s:e], acc[0:1])
                for s, e in self._runs(lambda m: m.tp_dim is None):
                    K.sumsq(self.grad[s:e], acc[1:2])
                t = (acc[0] + acc[1] / tp.size).view(1)
            else:
                K.sumsq(self.grad, acc[0:1])
                t = acc[0:1]
            if self.mesh.shard.size > 1:
                dist.all_reduce(t, group=self.mesh.shard.pg)
            if tp.size > 1:
                dist.all_reduce(t, group=tp.pg)
            return t[0].float()
        total = torch.zeros((), dtype=torch.float64, device=self.device)
        if tp.size > 1:
            sharded = torch.zeros((), dtype=torch.float64, device=self.device)
            for s, e in self._runs(lambda m: m.tp_dim is not None):
                sharded += self.grad[s:e].double().pow(2).sum()
            repl = torch.zeros((), dtype=torch.float64, device=self.device)
            for s, e in self._runs(lambda m: m.tp_dim is None):
                repl += self.grad[s:e].double().pow(2).sum()
            total = sharded + repl / tp.size
        else:
            total = self.grad.double().pow(2).sum()
        if self.mesh.shard.size > 1 or tp.size > 1:
            t = total.float().view(1)
            if self.mesh.shard.size > 1:
                dist.all_reduce(t, group=self.mesh.shard.pg)
            if tp.size > 1:
                dist.all_reduce(t, group=tp.pg)
            return t[0]
        return total.float()

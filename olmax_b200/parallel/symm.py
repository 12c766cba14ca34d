"""
Peer-memory ("fused") communication backend.

Replaces the collectives XLA inserts for the reference's shardings (all-gather of dim-0 sharded parameters, reduce-
scatter of their gradients: ``olmax/distributed/parallel.py:97-144,309-334``; explicit forms ``:409-436``) and fixes the
known issue that HSDP with gradient accumulation all-reduces after every micro-batch (``README.md:30`` of the reference).

The bf16 compute copy of the parameters and the fp32 gradient accumulator are allocated in symmetric memory
(``torch.distributed._symmetric_memory``: every rank of the job maps every other rank's buffer over NVLink), which
lets our kernels fuse the collectives into the compute instead of calling NCCL:

* **all-gather -> GEMM**: a weight is never gathered by a separate collective.  Every GEMM launch carries, in its copy
  warps, a slice of the NEXT FSDP unit's remote shards (so the transfer of layer i+1 runs under the math of layer i);
  whatever a weight still misses when its own GEMM starts is fetched by that GEMM itself, whose tiles then wait on
  per-block arrival counters (``csrc/gemm.cu``).  The embedding gather reads rows straight from the owner GPU.
* **GEMM -> reduce-scatter**: the weight-gradient GEMM's epilogue stores each row block (line-coalesced plain stores)
  into this rank's slot of the owner GPU's staging buffer; after one barrier per FSDP unit the owner folds its slots
  into its fp32 accumulator (scaled by 1 / (ranks x micro-batches)).  No atomics, deterministic summation order.
* **HSDP / DDP all-reduce**: once per optimizer step a two-shot kernel sums the fp32 accumulator over the replicas
  (plain peer loads / stores, or ``multimem.ld_reduce`` + ``multimem.st`` through NVSwitch when the group is the whole
  job and a multicast mapping exists).

Only plain loads / stores / reductions and multimem instructions touch peer memory; TMA descriptors always point at
local memory.  Stream-ordered barriers separate the phases (before the optimizer step: every peer's reductions have
landed and nobody still reads our weights; after it: every peer's new weights are visible and its accumulator is
cleared); the kernels themselves never wait on a peer except for the bounded arrival-counter wait inside one GEMM.
"""

from __future__ import annotations

import logging
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from ..ops import kernels as K

__all__ = ["SymmContext", "TPSymmContext", "symm_available"]

log = logging.getLogger(__name__)


def symm_available(device: torch.device) -> bool:
    if device.type != "cuda" or not dist.is_available() or not dist.is_initialized():
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return dist.get_backend() == "nccl"


class PeerBarrier:
    """
    Stream-ordered barrier over the GPUs ``ranks`` (global ranks).  Default: peer-mapped flag words
    (``ob_peer_barrier``), one small kernel per member that publishes an epoch in every member's flag array and waits
    for all of them, so the peer-memory path issues no library collective between its phases.
    ``OLMAX_B200_BARRIER=nccl``: a one-element NCCL all-reduce on ``pg`` instead (measured equal in step time: the cost
    of a barrier is the skew between ranks, not its latency).  Every wait of the flag barrier is bounded
    (``OLMAX_B200_BARRIER_TIMEOUT_S``, default 600 s, the order of NCCL's own watchdog: ranks may legitimately be far
    apart, e.g. while one of them writes a checkpoint): a member that never arrives makes the others record an error
    that ``ops._lib.check_status`` raises, the GPUs stay usable.  Construction is collective over the whole job.
    """

    def __init__(self, ranks: List[int], my_index: int, pg, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self.n, self.me, self.pg = len(ranks), my_index, pg
        self.use_flags = os.environ.get("OLMAX_B200_BARRIER", "flags") == "flags" and self.n <= 64
        self.timeout_s = float(os.environ.get("OLMAX_B200_BARRIER_TIMEOUT_S", "600"))
        self.epoch = 0
        self._last_waited = 0   # newest epoch this rank has waited for (debug check)
        self._token = torch.zeros(1, dtype=torch.float32, device=device)
        self._flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._h = symm_mem.rendezvous(self._flags, dist.group.WORLD)
        self._table = K.pointer_table([int(self._h.buffer_ptrs[r]) for r in ranks], device)
        # nobody may publish an epoch before every member has cleared its flags
        dist.all_reduce(self._token)
        torch.cuda.synchronize(device)

    def __call__(self) -> None:
        if self.n <= 1:
            return
        if not self.use_flags:
            dist.all_reduce(self._token, group=self.pg)
            return
        self.epoch += 1
        self._last_waited = self.epoch
        K.peer_barrier(self._table, self.me, self.n, self.epoch, self.timeout_s)

    # Split-phase use: ``token = arrive()`` when this rank's stores are done, ``wait(token)`` right before the others'
    # stores are needed; the skew between the ranks is then absorbed by whatever runs in between.
    def arrive(self):
        if self.n <= 1:
            return None
        if not self.use_flags:
            dist.all_reduce(self._token, group=self.pg)   # a collective cannot be split: the whole barrier happens here
            return None
        self.epoch += 1
        K.peer_signal(self._table, self.me, self.n, self.epoch)
        return self.epoch

    def wait(self, token) -> None:
        if token is not None:
            self._last_waited = max(self._last_waited, token)
            K.peer_wait(self._table, self.me, self.n, token, self.timeout_s)

    def check_flags(self) -> None:
        """Debug check (synchronises): after this rank's last barrier / wait every member's word in this rank's flag
        array must be the current epoch or one of the few a member may have published since (members run at most a
        handful of publishes ahead), never an older or a far newer one: a word outside that window means a member
        skipped a barrier, ran one twice, or a stray store hit the array."""
        if self.n <= 1 or not self.use_flags:
            return
        torch.cuda.synchronize(self._flags.device)
        words = self._flags[: self.n].tolist()
        for r, w in enumerate(words):
            if not (self._last_waited <= w <= self.epoch + 8):
                raise RuntimeError(f"barrier flag of member {r} is {w}; this rank last waited for {self._last_waited} and has "
                                   f"published {self.epoch}")
        if any(self._flags[self.n:].tolist()):
            raise RuntimeError("words of the flag array beyond the group size were written")


class SymmContext:
    N_STAGE = 3   # reduce-scatter staging buffers in rotation
    GUARD = 256   # guard words (fp32) on either side of the staging area
    CANARY = -7.25e22

    def __init__(self, store, numel: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.store = store
        mesh = store.mesh
        dev = store.device
        self.shadow = symm_mem.empty(numel, dtype=store.compute_dtype, device=dev)
        self.grad = symm_mem.empty(numel, dtype=torch.float32, device=dev)
        self.shadow.zero_()
        self.grad.zero_()
        world = dist.group.WORLD
        self._h_shadow = symm_mem.rendezvous(self.shadow, world)
        self._h_grad = symm_mem.rendezvous(self.grad, world)
        all_shadow = [int(p) for p in self._h_shadow.buffer_ptrs]
        all_grad = [int(p) for p in self._h_grad.buffer_ptrs]
        # the shard group's view (index = rank inside the shard group)
        self.R = mesh.shard.size
        self.rank = mesh.shard.rank
        self.shadow_ptrs: List[int] = [all_shadow[r] for r in mesh.shard.ranks]
        self.grad_ptrs: List[int] = [all_grad[r] for r in mesh.shard.ranks]
        # the replicate group's view, for the once-per-step gradient all-reduce
        self.replica_grad_table = K.pointer_table([all_grad[r] for r in mesh.replicate.ranks], dev)
        mc = int(getattr(self._h_grad, "multicast_ptr", 0) or 0)
        use_mc = os.environ.get("OLMAX_B200_MULTIMEM", "1") == "1"
        self.multicast_ptr = mc if (use_mc and mesh.replicate.size == mesh.world_size) else 0
        # Reduce-scatter staging: every weight-gradient GEMM STORES (plain stores, no atomics) the row block owned by
        # GPU r into slot `me` of r's staging buffer; r folds its R slots into its accumulator once every member has
        # published that its stores of that unit are done.  The fold of unit u is deferred to the moment unit u-1 (the
        # next one in backward order) has been computed: [wgrads(u-1)] -> wait(u) -> fold(u) -> publish(u-1), so the
        # wait finds the others' epoch already there unless they lag by more than a whole unit.  Three buffers rotate
        # (index % 3): a buffer is written again for unit u-3 only after this rank has passed wait(u-1), and a member
        # publishes (u-1) only after its fold(u), the previous user of that buffer.
        self.stage_slot = max((u.numel_local for u in store.units), default=0)
        self.stage_slot = (self.stage_slot + 7) // 8 * 8
        self.rs_stage = None
        self.stage_ptrs: List[int] = []
        # Wire format of the staged partial gradients: bf16 (half the bytes over NVLink and in the fold; each rank's
        # partial sum is rounded once, the fold and the accumulator stay fp32; the reference reduces bf16 gradients
        # too, `olmax/train/trainer.py:728-739`) or fp32.  bf16 needs every parameter's local slice to start and end
        # on a multiple of 8 elements.
        wire = os.environ.get("OLMAX_B200_RS_WIRE", "bf16")
        if wire not in ("fp32", "bf16"):
            raise ValueError(f"OLMAX_B200_RS_WIRE must be fp32 or bf16, got {wire!r}")
        if wire == "bf16" and any(h.meta.unit_offset % 8 or h.meta.numel_local % 8 for u in store.units for h in u.params):
            log.warning("bf16 reduce-scatter wire needs 8-element aligned parameter slices; using fp32")
            wire = "fp32"
        self.wire_dtype = torch.bfloat16 if wire == "bf16" else torch.float32
        self.wire_bytes = 2 if wire == "bf16" else 4
        if self.R > 1 and os.environ.get("OLMAX_B200_FUSED_RS", "1") == "1":
            # guard words before and after the staging area: peers only ever store inside it (check_canaries)
            n_stage = self.N_STAGE * self.R * self.stage_slot
            self._stage_alloc = symm_mem.empty(n_stage + 2 * self.GUARD, dtype=self.wire_dtype, device=dev)
            self._stage_alloc[: self.GUARD] = self.CANARY
            self._stage_alloc[self.GUARD + n_stage:] = self.CANARY
            self.rs_stage = self._stage_alloc[self.GUARD : self.GUARD + n_stage]
            self._h_stage = symm_mem.rendezvous(self._stage_alloc, world)
            all_stage = [int(p) + self.GUARD * self.wire_bytes for p in self._h_stage.buffer_ptrs]
            self.stage_ptrs = [all_stage[r] for r in mesh.shard.ranks]
        self.flags = torch.zeros(max(1, self.R) * 4096, dtype=torch.int32, device=dev)
        self._rs_pending = None   # (unit, names, barrier token) of the unit whose fold is still to come
        self._tables: Dict[tuple, torch.Tensor] = {}
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        self._sync_group = world if mesh.replicate.size > 1 else mesh.shard.pg
        if mesh.replicate.size > 1:
            self._barrier = PeerBarrier(list(range(mesh.world_size)), mesh.rank, world, dev)
        else:
            self._barrier = PeerBarrier(list(mesh.shard.ranks), mesh.shard.rank, mesh.shard.pg, dev)
        log.info("Peer-memory backend on: shard group %d, replicate group %d, %.1f MiB bf16 weights + %.1f MiB fp32 "
                 "gradients mapped per rank%s", self.R, mesh.replicate.size, numel * 2 / 2**20, numel * 4 / 2**20,
                 ", NVLS multicast" if self.multicast_ptr else "")

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

    def stage_pointer_table(self, handle) -> torch.Tensor:
        """Device array: for every owner GPU r, the address inside r's staging buffer where THIS rank's contribution
        to the row shard r of ``handle``'s gradient goes (buffer chosen by the parity of the unit index)."""
        buf = handle.unit.index % self.N_STAGE
        key = ("stage", handle.name, buf)
        t = self._tables.get(key)
        if t is None:
            off = ((buf * self.R + self.rank) * self.stage_slot + handle.meta.unit_offset) * self.wire_bytes
            t = K.pointer_table([p + off for p in self.stage_ptrs], self.store.device)
            self._tables[key] = t
        return t

    def fold_stage(self, unit, names) -> None:
        """accumulator += grad_scale * sum over the R slots of the unit's staging buffer, for the parameters in
        ``names`` (those whose weight gradient was stored this pass; other regions of the slots hold stale data)."""
        buf = unit.index % self.N_STAGE
        base = buf * self.R * self.stage_slot
        for h in unit.params:
            if h.name not in names:
                continue
            m = h.meta
            stage = self.rs_stage[base + m.unit_offset:]
            acc = self.grad[m.offset : m.offset + m.numel_local]
            K.reduce_slots(stage, acc, m.numel_local, self.R, self.stage_slot, self.store.grad_scale)

    def check_canaries(self) -> None:
        """Debug check (synchronises): the guard words around this rank's reduce-scatter staging area are intact, i.e.
        no peer's weight-gradient epilogue stored outside the slots it owns; also checks the barrier's flag words."""
        torch.cuda.synchronize(self.store.device)
        if self.rs_stage is not None:
            g = self.GUARD
            lo, hi = self._stage_alloc[:g], self._stage_alloc[-g:]
            if not (bool((lo == self.CANARY).all()) and bool((hi == self.CANARY).all())):
                raise RuntimeError("guard words around the reduce-scatter staging buffer were overwritten")
        self._barrier.check_flags()

    def rs_unit_done(self, unit, names) -> None:
        """This rank has launched every weight-gradient GEMM of ``unit`` (their epilogues store into the owners'
        staging slots).  Folds the PREVIOUS unit's slots (waiting, normally without delay, for the members' epoch of
        that unit) and then publishes this unit's epoch; this unit is folded at the next call or by :meth:`rs_flush`."""
        self._fold_pending()
        self._rs_pending = (unit, names, self._barrier.arrive())

    def _fold_pending(self) -> None:
        if self._rs_pending is not None:
            unit, names, token = self._rs_pending
            self._rs_pending = None
            self._barrier.wait(token)
            self.fold_stage(unit, names)

    def rs_flush(self) -> None:
        """Fold whatever is still staged (end of a backward pass)."""
        self._fold_pending()

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
        """Stream-ordered barrier over every rank that shares memory with this one (:class:`PeerBarrier`)."""
        self._barrier()

    def all_reduce_replicas(self) -> int:
        """Sum the fp32 gradient accumulator over the replicate group with our peer-memory kernel; returns the bytes
        this rank moved over NVLink.  Barriers before and after are the caller's (``sync_peers``)."""
        rep = self.store.mesh.replicate
        n = self.grad.numel()
        if self.multicast_ptr and n % 4 == 0:
            K.allreduce_multimem(self.multicast_ptr, n, rep.rank, rep.size)
        else:
            K.allreduce_p2p(self.replica_grad_table, n, rep.rank, rep.size)
        return 2 * (rep.size - 1) * n * 4 // rep.size


class TPSymmContext:
    """
    Peer-memory buffers of a tensor-parallel group with sequence parallelism, for the two fused activation paths:

    * **all-gather -> GEMM**: ``gather_begin(x_local)`` copies this rank's rows into a symmetric buffer, passes a
      stream-ordered barrier and returns the full ``[M, d]`` activation with only the local rows filled plus the GEMM
      arguments that make the FIRST consuming GEMM pull the other rows from the peers with its copy warps while its
      tensor cores start on the local rows (``ag_on_a`` of ``csrc/gemm.h``).
    * **GEMM -> reduce-scatter**: ``rs_begin(M_s, N)`` returns the pointer table that makes a GEMM epilogue store row
      block s of its partial product into this rank's slot of GPU s's staging buffer; ``rs_finish`` passes a barrier and
      folds the slots into the local ``[M_s, N]`` result.

    Buffers alternate between two copies.  Every publish / staging buffer is reused only after a later barrier of the
    same group, which every member passes after the kernels that read (or wrote) the buffer: gather and reduce-scatter
    regions alternate in a transformer (each block is entered by a gather and left by a reduce-scatter, in forward,
    recomputation and backward alike), so between two uses of a buffer there are at least two such barriers.
    """

    def __init__(self, mesh, device: torch.device):
        self.mesh = mesh
        self.group = mesh.tp
        self.n = mesh.tp.size
        self.rank = mesh.tp.rank
        self.device = device
        self._x: Dict[int, list] = {}       # capacity (elements) -> [(tensor, pointer table of the group's buffers)] * 2
        self._stage: Dict[int, list] = {}   # slot elements -> [(tensor [n * slot], table of "my slot on GPU s")] * 2
        self._flip_x = 0
        self._flip_s = 0
        self.flags = torch.zeros(self.n * 4096, dtype=torch.int32, device=device)
        self._barrier = PeerBarrier(list(self.group.ranks), self.rank, self.group.pg, device)
        self.bytes_gathered = 0
        self.bytes_scattered = 0
        # OLMAX_B200_TP_AG: how the row shards of a gathered activation reach this GPU.
        #   copy (default): our copy kernel pulls them from the peers' buffers before the consuming GEMM (remote loads
        #                   at ~640 GB/s per direction on this hardware);
        #   gemm:           the consuming GEMM's copy warps pull them while its tensor cores work on the local rows
        #                   (measured slower: the copy warps' loads starve next to the GEMM's own operand traffic);
        #   nccl:           NCCL all-gather.
        # OLMAX_B200_TP_RS=nccl reduce-scatters a row-parallel output with NCCL after the GEMM instead of in its epilogue.
        self.ag_mode = os.environ.get("OLMAX_B200_TP_AG", "copy")
        if self.ag_mode not in ("copy", "gemm", "nccl"):
            raise ValueError(f"OLMAX_B200_TP_AG={self.ag_mode!r}: expected copy, gemm or nccl")
        self.rs_in_gemm = os.environ.get("OLMAX_B200_TP_RS", "gemm") == "gemm"
        log.info("Tensor-parallel peer-memory context: group of %d (rank %d)", self.n, self.rank)

    def _symm_pair(self, numel: int, slot_offset_elems: int):
        """Two symmetric bf16 buffers of ``numel`` elements and, for each, the device table of the addresses
        ``peer buffer + slot_offset_elems`` over the TP group.  Collective over the whole job (same order everywhere)."""
        import torch.distributed._symmetric_memory as symm_mem

        out = []
        for _ in range(2):
            t = symm_mem.empty(numel, dtype=torch.bfloat16, device=self.device)
            t.zero_()
            h = symm_mem.rendezvous(t, dist.group.WORLD)
            ptrs = [int(p) for p in h.buffer_ptrs]
            addrs = [ptrs[r] + slot_offset_elems * 2 for r in self.group.ranks]
            out.append((t, K.pointer_table(addrs, self.device), addrs))
        return out

    def barrier(self) -> None:
        self._barrier()

    def stats_buffer(self, numel: int, index: int):
        """(fp32 tensor of ``numel`` elements in symmetric memory, device table of the group's addresses of that
        buffer) for small per-row statistics exchanged between the members (vocabulary-parallel cross entropy).  Two
        buffers alternate with ``index``: a buffer is written again only after a later barrier of the group, which every
        member passes after the kernel that read the previous contents."""
        import torch.distributed._symmetric_memory as symm_mem

        key = ("stats", numel)
        if key not in self._x:
            pair = []
            for _ in range(2):
                t = symm_mem.empty(numel, dtype=torch.float32, device=self.device)
                t.zero_()
                h = symm_mem.rendezvous(t, dist.group.WORLD)
                ptrs = [int(p) for p in h.buffer_ptrs]
                pair.append((t, K.pointer_table([ptrs[r] for r in self.group.ranks], self.device)))
            self._x[key] = pair
        return self._x[key][index & 1]

    # ---- all-gather -> GEMM -----------------------------------------------------------------------------------------
    def gather_begin(self, x_local: torch.Tensor):
        """x_local [M_s, d] bf16 -> (x_full [M, d] with rows of this rank filled, kwargs for the first consuming GEMM)."""
        M_s, d = x_local.shape
        numel = M_s * d
        if self.ag_mode == "nccl":
            from . import collectives as coll

            with K.timed_region("nccl seq all_gather"):
                return coll.all_gather(x_local, self.group, dim=0), {}
        if numel not in self._x:
            self._x[numel] = self._symm_pair(numel, 0)
        buf, table, addrs = self._x[numel][self._flip_x]
        self._flip_x ^= 1
        with K.timed_region("tp publish copies"):
            buf.view(M_s, d).copy_(x_local)
            x_full = torch.empty((self.n * M_s, d), dtype=x_local.dtype, device=x_local.device)
            x_full[self.rank * M_s : (self.rank + 1) * M_s].copy_(x_local)
        self.barrier()   # every member's rows are in its buffer before anybody's GEMM pulls them
        self.bytes_gathered += (self.n - 1) * numel * 2
        if self.ag_mode == "copy":
            for ds in range(1, self.n):   # peers in the order rank+1, rank+2, ...: no two GPUs start on the same source
                s = (self.rank + ds) % self.n
                K.copy_bytes(x_full.data_ptr() + s * numel * 2, addrs[s], numel * 2, self.device, unroll=8)
            return x_full, {}
        return x_full, {"ag_src": table, "ag_flags": self.flags, "ag_rank": self.rank, "ag_on_a": True, "M_s": M_s}

    def finish_gather(self, x_full: torch.Tensor, kw: dict) -> None:
        """Complete a gather that no GEMM consumed (``kw`` from ``gather_begin``)."""
        if kw:
            numel = x_full.numel() // self.n
            K.gather_shards(kw["ag_src"], x_full, numel, numel, self.n, self.rank)

    # ---- GEMM -> reduce-scatter -------------------------------------------------------------------------------------
    def rs_begin(self, M_s: int, N: int):
        """(staging tensor, kwargs for the GEMM whose [n * M_s, N] output is to be reduce-scattered)."""
        slot = M_s * N
        if not self.rs_in_gemm:
            full = torch.empty((self.n * M_s, N), dtype=torch.bfloat16, device=self.device)
            return full, {}
        if slot not in self._stage:
            self._stage[slot] = self._symm_pair(self.n * slot, self.rank * slot)
        buf, table, _addrs = self._stage[slot][self._flip_s]
        self._flip_s ^= 1
        # the peers' row blocks are computed first so that their transfer starts early; the local block comes last
        return buf, {"M_s": M_s, "c_shards": table, "m_shard_rot": (self.rank + 1) % self.n}

    def rs_finish(self, stage: torch.Tensor, M_s: int, N: int) -> torch.Tensor:
        if not self.rs_in_gemm:
            from . import collectives as coll

            return coll.reduce_scatter(stage, self.group, dim=0)
        self.barrier()   # every member's stores into our slots have completed
        out = torch.empty((M_s, N), dtype=torch.bfloat16, device=self.device)
        K.fold_slots_bf16(out, stage, M_s * N, self.n, M_s * N, skip=-1, accumulate=False)
        self.bytes_scattered += (self.n - 1) * M_s * N * 2
        return out

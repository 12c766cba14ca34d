"""
Device mesh description and the parallelism configs (role of ``olmax/distributed/parallel.py:20-455``).

:class:`MeshResource` names the mesh axes and says which axis shards the batch, the parameters (FSDP), the hidden
dimension (TP) and the sequence (CP).  It is pure data and can be built without a process group (so configs can be
printed and validated anywhere).  :meth:`MeshResource.build` turns it into a :class:`DeviceMesh`: this rank's
coordinates plus one ``torch.distributed`` process group per axis, which is what the sharding layer and the
collectives use.

Ranks are laid out row-major over the axes (the last axis varies fastest), so with ``HSDP`` the ranks of one shard
group are consecutive (one NVLink domain) and with ``FSDP_with_TP`` the two ranks of a TP pair are neighbours.
"""

from __future__ import annotations

import dataclasses
import itertools
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from ..exceptions import OLMaxConfigurationError
from ..types import StrEnum
from . import dist_utils

__all__ = [
    "shard_map",
    "TPStyle",
    "DataParallelType",
    "DataParallelConfig",
    "TensorParallelConfig",
    "ContextParallelConfig",
    "PipelineParallelConfig",
    "ExpertParallelConfig",
    "MeshResource",
    "DeviceMesh",
    "get_mesh",
    "set_mesh",
]

AxisSpec = Union[str, Tuple[str, ...], None]


class TPStyle(StrEnum):
    """How a Linear is split over the tensor-parallel axis: output features (colwise) or input features (rowwise)."""

    colwise = "colwise"
    rowwise = "rowwise"


class DataParallelType(StrEnum):
    fsdp = "fsdp"
    hsdp = "hsdp"
    ddp = "ddp"


@dataclass(frozen=True)
class DataParallelConfig:
    name: DataParallelType = DataParallelType.fsdp
    shard_degree: Optional[int] = None

    def build_mesh(self, world_size: Optional[int] = None, tp: Optional["TensorParallelConfig"] = None) -> "MeshResource":
        tp_degree = tp.degree if tp is not None else 1
        if self.name == DataParallelType.ddp:
            return MeshResource.DDP(world_size)
        if self.name == DataParallelType.hsdp:
            return MeshResource.HSDP(self.shard_degree, world_size)
        if tp_degree > 1:
            return MeshResource.FSDP_with_TP(tp_degree, world_size)
        return MeshResource.FSDP(world_size)


@dataclass(frozen=True)
class TensorParallelConfig:
    degree: int = 1
    sequence_parallel: bool = True


@dataclass(frozen=True)
class ContextParallelConfig:
    degree: int = 1
    use_dp_shard_axis: bool = False


@dataclass(frozen=True)
class PipelineParallelConfig:
    """Declared for config compatibility; no pipeline schedule exists (neither does one in the reference)."""

    degree: int = 1


@dataclass(frozen=True)
class ExpertParallelConfig:
    """Declared for config compatibility; there is no MoE layer (neither is there one in the reference)."""

    degree: int = 1


def _world(global_device_count: Optional[int]) -> int:
    return global_device_count if global_device_count is not None else dist_utils.get_global_device_count()


@dataclass(frozen=True)
class MeshResource:
    axes: Tuple[Tuple[int, str], ...]
    """``(axis_size, axis_name)`` pairs, outermost first."""
    batch_sharding_axis: AxisSpec = None
    fsdp_sharding_axis: AxisSpec = None
    tp_sharding_axis: Optional[str] = None
    cp_sharding_axis: Optional[str] = None

    def __post_init__(self):
        # tolerate lists / 3-tuples (size, name, axis_type) coming from decoded configs
        norm = tuple((int(a[0]), str(a[1])) for a in self.axes)
        object.__setattr__(self, "axes", norm)
        for spec_name in ("batch_sharding_axis", "fsdp_sharding_axis"):
            spec = getattr(self, spec_name)
            if isinstance(spec, list):
                object.__setattr__(self, spec_name, tuple(spec))
        names = [n for _, n in norm]
        if len(set(names)) != len(names):
            raise OLMaxConfigurationError(f"duplicate mesh axis names: {names}")
        for spec in (self.batch_sharding_axis, self.fsdp_sharding_axis, self.tp_sharding_axis, self.cp_sharding_axis):
            for ax in self._as_tuple(spec):
                if ax not in names:
                    raise OLMaxConfigurationError(f"axis '{ax}' is not part of the mesh {names}")

    # ------------------------------------------------------------------ factories
    @classmethod
    def FSDP(cls, global_device_count: Optional[int] = None) -> "MeshResource":
        return cls(axes=((_world(global_device_count), "fsdp"),), batch_sharding_axis="fsdp", fsdp_sharding_axis="fsdp")

    @classmethod
    def HSDP(
        cls,
        shard_degree: Optional[int] = None,
        global_device_count: Optional[int] = None,
        local_device_count: Optional[int] = None,
    ) -> "MeshResource":
        world = _world(global_device_count)
        if shard_degree is None or shard_degree < 0:
            shard_degree = local_device_count if local_device_count is not None else dist_utils.get_local_device_count()
        if shard_degree <= 0 or world % shard_degree != 0:
            raise OLMaxConfigurationError(f"shard degree {shard_degree} does not divide {world} devices")
        return cls(
            axes=((world // shard_degree, "fsdp_replicate"), (shard_degree, "fsdp_shard")),
            batch_sharding_axis=("fsdp_replicate", "fsdp_shard"),
            fsdp_sharding_axis="fsdp_shard",
        )

    @classmethod
    def DDP(cls, global_device_count: Optional[int] = None) -> "MeshResource":
        return cls(axes=((_world(global_device_count), "data"),), batch_sharding_axis="data", fsdp_sharding_axis=None)

    @classmethod
    def FSDP_with_TP(cls, tp_degree: int, global_device_count: Optional[int] = None) -> "MeshResource":
        world = _world(global_device_count)
        if tp_degree <= 0 or world % tp_degree != 0:
            raise OLMaxConfigurationError(f"tp degree {tp_degree} does not divide {world} devices")
        return cls(
            axes=((world // tp_degree, "fsdp"), (tp_degree, "tp")),
            batch_sharding_axis="fsdp",
            fsdp_sharding_axis="fsdp",
            tp_sharding_axis="tp",
        )

    @classmethod
    def FSDP_with_CP(cls, global_device_count: Optional[int] = None, cp_degree: int = -1) -> "MeshResource":
        world = _world(global_device_count)
        if cp_degree < 0:
            return cls(axes=((world, "context"),), batch_sharding_axis=None, fsdp_sharding_axis="context",
                       cp_sharding_axis="context")
        if cp_degree == 0 or world % cp_degree != 0:
            raise OLMaxConfigurationError(f"cp degree {cp_degree} does not divide {world} devices")
        return cls(
            axes=((world // cp_degree, "batch"), (cp_degree, "context")),
            batch_sharding_axis="batch",
            fsdp_sharding_axis=("batch", "context"),
            cp_sharding_axis="context",
        )

    @classmethod
    def HSDP_with_CP(
        cls,
        shard_degree: Optional[int] = None,
        global_device_count: Optional[int] = None,
        local_device_count: Optional[int] = None,
    ) -> "MeshResource":
        base = cls.HSDP(shard_degree, global_device_count, local_device_count)
        return dataclasses.replace(base, batch_sharding_axis="fsdp_replicate", cp_sharding_axis="fsdp_shard")

    # ------------------------------------------------------------------ queries
    @staticmethod
    def _as_tuple(spec: AxisSpec) -> Tuple[str, ...]:
        if spec is None:
            return ()
        if isinstance(spec, str):
            return (spec,)
        return tuple(spec)

    @property
    def axis_shapes(self) -> Tuple[int, ...]:
        return tuple(s for s, _ in self.axes)

    @property
    def axis_names(self) -> Tuple[str, ...]:
        return tuple(n for _, n in self.axes)

    @property
    def size(self) -> int:
        n = 1
        for s in self.axis_shapes:
            n *= s
        return n

    def axis_size(self, axis: Union[int, str, Tuple[str, ...], None]) -> int:
        if axis is None:
            return 1
        if isinstance(axis, int):
            return self.axis_shapes[axis]
        n = 1
        for ax in self._as_tuple(axis):
            n *= self.axis_shapes[self.axis_names.index(ax)]
        return n

    def has_axis(self, axis: str) -> bool:
        return axis in self.axis_names

    @property
    def data_parallel_size(self) -> int:
        """Number of distinct data shards = devices / (cp * tp)."""
        return self.size // (self.axis_size(self.cp_sharding_axis) * self.axis_size(self.tp_sharding_axis))

    @property
    def fsdp_size(self) -> int:
        return self.axis_size(self.fsdp_sharding_axis)

    @property
    def tp_size(self) -> int:
        return self.axis_size(self.tp_sharding_axis)

    @property
    def cp_size(self) -> int:
        return self.axis_size(self.cp_sharding_axis)

    @property
    def replicate_axes(self) -> Tuple[str, ...]:
        """Axes over which parameters are replicated and gradients therefore all-reduced (data axes not used by
        FSDP, e.g. ``fsdp_replicate`` under HSDP or ``data`` under DDP)."""
        fsdp = set(self._as_tuple(self.fsdp_sharding_axis))
        skip = fsdp | set(self._as_tuple(self.tp_sharding_axis))
        batch = self._as_tuple(self.batch_sharding_axis)
        return tuple(a for a in batch if a not in skip)

    def coordinates(self, rank: int) -> Dict[str, int]:
        coords = {}
        rem = rank
        for size, name in reversed(self.axes):
            coords[name] = rem % size
            rem //= size
        return coords

    def rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for size, name in self.axes:
            r = r * size + coords[name]
        return r

    def group_ranks(self, axes: AxisSpec, rank: int) -> List[int]:
        """Ranks that differ from ``rank`` only along ``axes`` (ordered by their coordinates on those axes)."""
        names = self._as_tuple(axes)
        base = self.coordinates(rank)
        sizes = [self.axis_size(n) for n in names]
        out = []
        for combo in itertools.product(*[range(s) for s in sizes]):
            c = dict(base)
            for n, v in zip(names, combo):
                c[n] = v
            out.append(self.rank_of(c))
        return out

    def build(self, device: Optional[torch.device] = None) -> "DeviceMesh":
        return DeviceMesh(self, device=device)

    def describe(self) -> str:
        axes = " x ".join(f"{n}={s}" for s, n in self.axes)
        return (f"Mesh({axes}; batch={self.batch_sharding_axis}, fsdp={self.fsdp_sharding_axis}, "
                f"tp={self.tp_sharding_axis}, cp={self.cp_sharding_axis})")


class _Group:
    """A process group plus its rank list; ``pg`` is None for a group of one."""

    def __init__(self, ranks: List[int], my_rank: int, pg: Optional[dist.ProcessGroup]):
        self.ranks = ranks
        self.size = len(ranks)
        self.rank = ranks.index(my_rank)
        self.pg = pg

    def __repr__(self) -> str:
        return f"Group(size={self.size}, rank={self.rank}, ranks={self.ranks})"


class DeviceMesh:
    """
    Runtime view of a :class:`MeshResource` for this process: coordinates and process groups.

    Groups are created for the FSDP shard axes, the replicate axes, the TP axis, the CP axis and the full batch axes.
    Creation is collective: every rank of the job must construct the DeviceMesh at the same point.
    """

    def __init__(self, resource: MeshResource, device: Optional[torch.device] = None):
        world = dist_utils.get_world_size()
        if resource.size != world:
            raise OLMaxConfigurationError(f"{resource.describe()} needs {resource.size} processes, job has {world}")
        self.resource = resource
        self.rank = dist_utils.get_rank()
        self.world_size = world
        self.device = device if device is not None else dist_utils.get_device()
        self.coords = resource.coordinates(self.rank)
        self._groups: Dict[Tuple[str, ...], _Group] = {}
        self.shard = self._make_group(resource.fsdp_sharding_axis)
        self.replicate = self._make_group(resource.replicate_axes or None)
        self.tp = self._make_group(resource.tp_sharding_axis)
        self.cp = self._make_group(resource.cp_sharding_axis)
        self.batch = self._make_group(resource.batch_sharding_axis)
        self.world = self._make_group(tuple(resource.axis_names))

    def _make_group(self, axes: AxisSpec) -> _Group:
        names = MeshResource._as_tuple(axes)
        if names in self._groups:
            return self._groups[names]
        if not names or self.world_size == 1:
            g = _Group([self.rank], self.rank, None)
            self._groups[names] = g
            return g
        # every rank creates every group of this axis set, in the same order (new_group is collective)
        seen = set()
        mine: Optional[_Group] = None
        for r in range(self.world_size):
            ranks = tuple(self.resource.group_ranks(names, r))
            if ranks in seen:
                continue
            seen.add(ranks)
            if len(ranks) == self.world_size:
                pg = dist.group.WORLD
            elif len(ranks) == 1:
                pg = None
            else:
                pg = dist.new_group(ranks=list(ranks))
            if self.rank in ranks:
                mine = _Group(list(ranks), self.rank, pg)
        assert mine is not None
        self._groups[names] = mine
        return mine

    @property
    def data_parallel_rank(self) -> int:
        """Index of this rank's data shard in [0, data_parallel_size)."""
        res = self.resource
        skip = set(MeshResource._as_tuple(res.tp_sharding_axis)) | set(MeshResource._as_tuple(res.cp_sharding_axis))
        idx = 0
        for size, name in res.axes:
            if name in skip:
                continue
            idx = idx * size + self.coords[name]
        return idx

    @property
    def data_parallel_size(self) -> int:
        return self.resource.data_parallel_size

    def describe(self) -> str:
        return f"{self.resource.describe()} rank={self.rank} coords={self.coords}"


_CURRENT: Optional[DeviceMesh] = None


def set_mesh(mesh: Optional[DeviceMesh]) -> None:
    global _CURRENT
    _CURRENT = mesh


def get_mesh() -> Optional[DeviceMesh]:
    return _CURRENT


def shard_map(fun, mesh: Optional[DeviceMesh] = None, in_specs=None, out_specs=None, **_ignored):
    """Counterpart of the reference's ``shard_map`` wrapper (``olmax/distributed/parallel.py:404-407``).  Under JAX it
    turns a function over global arrays into a per-shard function; with one process per device every function already
    runs on this rank's shards and calls the collectives of :mod:`olmax_b200.parallel.collectives` explicitly, so the
    function is returned unchanged (the specs are accepted so that call sites keep their shape)."""
    return fun

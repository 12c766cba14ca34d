"""
Process bootstrap and host-level synchronisation (role of ``olmax/distributed/utils.py:18-214``).

One process per GPU.  ``init_distributed`` creates the default process group (NCCL when CUDA is available, gloo
otherwise) and, next to it, a gloo group for control-plane traffic (barriers, cancellation flags, small Python
values), so host synchronisation never enqueues work on a GPU.  Without an initialised process group every query
degrades to the single-process answer, which lets library code run unchanged in unit tests.
"""

from __future__ import annotations

import datetime
import logging
import os
from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from ..exceptions import OLMaxEnvironmentError

__all__ = [
    "DistConfig",
    "init_distributed",
    "teardown_distributed",
    "is_distributed",
    "get_rank",
    "get_world_size",
    "get_local_rank",
    "get_local_device_count",
    "get_global_device_count",
    "get_process_count",
    "get_process_index",
    "get_process_filesystem_rank",
    "get_device",
    "control_group",
    "barrier",
    "synchronize_value",
    "synchronize_array",
    "allgather_value",
    "get_reduce_divide_factor",
]

log = logging.getLogger(__name__)

_CONTROL_GROUP: Optional[dist.ProcessGroup] = None
_OWNS_PG = False
_FS_RANK_CACHE: Optional[int] = None


@dataclass
class DistConfig:
    """
    Rendezvous description.  Fields left as None are read from the torchrun-style environment
    (``MASTER_ADDR``, ``MASTER_PORT``, ``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``).
    """

    coordinator_address: Optional[str] = None  # "host:port"
    num_processes: Optional[int] = None
    process_id: Optional[int] = None
    local_rank: Optional[int] = None
    backend: Optional[str] = None  # default: nccl with CUDA, gloo without
    initialization_timeout: int = 300  # seconds

    @classmethod
    def from_env(cls) -> Optional["DistConfig"]:
        if "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
            return None
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = os.environ.get("MASTER_PORT", "29400")
        return cls(
            coordinator_address=f"{addr}:{port}",
            num_processes=int(os.environ["WORLD_SIZE"]),
            process_id=int(os.environ["RANK"]),
            local_rank=int(os.environ.get("LOCAL_RANK", os.environ["RANK"])),
        )


def init_distributed(config: Optional[DistConfig] = None) -> None:
    """Join the job-wide process group (no-op for a single process without a rendezvous environment)."""
    global _CONTROL_GROUP, _OWNS_PG
    if dist.is_available() and dist.is_initialized():
        if _CONTROL_GROUP is None and dist.get_world_size() > 1:
            _CONTROL_GROUP = dist.new_group(backend="gloo")
        return
    if config is None:
        config = DistConfig.from_env()
    if config is None or (config.num_processes or 1) <= 1 and config.coordinator_address is None:
        return
    if config.coordinator_address is None or config.num_processes is None or config.process_id is None:
        raise OLMaxEnvironmentError("DistConfig needs coordinator_address, num_processes and process_id")
    use_cuda = torch.cuda.is_available()
    backend = config.backend or ("nccl" if use_cuda else "gloo")
    local_rank = config.local_rank if config.local_rank is not None else config.process_id
    os.environ.setdefault("LOCAL_RANK", str(local_rank))
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    host, _, port = config.coordinator_address.rpartition(":")
    kwargs = {}
    if backend == "nccl" and use_cuda:
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(
        backend=backend,
        init_method=f"tcp://{host}:{port}",
        world_size=config.num_processes,
        rank=config.process_id,
        timeout=datetime.timedelta(seconds=config.initialization_timeout),
        **kwargs,
    )
    _OWNS_PG = True
    if backend != "gloo":
        _CONTROL_GROUP = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=config.initialization_timeout))
    log.info("Joined process group: rank %d of %d (backend %s)", get_rank(), get_world_size(), backend)


def teardown_distributed() -> None:
    global _CONTROL_GROUP, _OWNS_PG, _FS_RANK_CACHE
    _FS_RANK_CACHE = None
    if dist.is_available() and dist.is_initialized() and _OWNS_PG:
        try:
            dist.destroy_process_group()
        finally:
            _CONTROL_GROUP = None
            _OWNS_PG = False


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", get_rank()))


def get_local_device_count() -> int:
    """Devices driven from this host (``LOCAL_WORLD_SIZE`` under a launcher, else visible GPUs, else 1)."""
    if "LOCAL_WORLD_SIZE" in os.environ:
        return int(os.environ["LOCAL_WORLD_SIZE"])
    if torch.cuda.is_available():
        return min(torch.cuda.device_count(), get_world_size()) or 1
    return get_world_size()


def get_global_device_count() -> int:
    """One device per process."""
    return get_world_size()


def get_process_count() -> int:
    return get_world_size()


def get_process_index() -> int:
    return get_rank()


def get_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def control_group() -> Optional[dist.ProcessGroup]:
    """The CPU (gloo) group used for host-side synchronisation; None when not distributed."""
    if not is_distributed():
        return None
    if _CONTROL_GROUP is not None:
        return _CONTROL_GROUP
    if dist.get_backend() == "gloo":
        return dist.group.WORLD
    return None


def get_process_filesystem_rank() -> int:
    """
    Rank among the processes that share this process's file system: 0 is the one that should write shared files.
    Directories listed in ``OLMAX_SHARED_FS_DIRS`` (colon separated) are treated as shared by every rank, otherwise
    each host is its own file system and the local rank decides (``olmax/distributed/utils.py:101-156``).
    """
    global _FS_RANK_CACHE
    if _FS_RANK_CACHE is not None:
        return _FS_RANK_CACHE
    if os.environ.get("OLMAX_SHARED_FS_DIRS"):
        _FS_RANK_CACHE = get_rank()
    else:
        _FS_RANK_CACHE = get_local_rank()
    return _FS_RANK_CACHE


def barrier(name: str = "barrier") -> None:
    """Host barrier over the control group (never touches a GPU)."""
    del name
    if not is_distributed():
        return
    group = control_group()
    if group is not None:
        dist.barrier(group=group)
    else:
        dist.barrier()


def synchronize_value(value: Any, src: int = 0) -> Any:
    """Every rank gets rank ``src``'s Python value."""
    if not is_distributed():
        return value
    box: List[Any] = [value if get_rank() == src else None]
    dist.broadcast_object_list(box, src=src, group=control_group())
    return box[0]


def synchronize_array(x: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Every rank gets rank ``src``'s tensor (broadcast over the control group for CPU tensors)."""
    if not is_distributed():
        return x
    if x.is_cuda:
        dist.broadcast(x, src=src)
        return x
    dist.broadcast(x, src=src, group=control_group())
    return x


def allgather_value(value: Any) -> List[Any]:
    if not is_distributed():
        return [value]
    out: List[Any] = [None] * get_world_size()
    dist.all_gather_object(out, value, group=control_group())
    return out


def get_reduce_divide_factor(n: int) -> int:
    """
    Pre-divide factor for low-precision sums over ``n`` ranks: the smallest power of two ``f`` with ``f >= n / f``
    (2->2, 4->2, 8->4, 16->4, 32->8, 64->8).  Dividing by ``f`` before and by ``n / f`` after the sum keeps bf16
    partial sums in range (``olmax/distributed/utils.py:210-214``).
    """
    f = 1
    while n % f == 0 and n / f > f:
        f *= 2
    return f

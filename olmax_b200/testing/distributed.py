"""
Multi-process test harness (``olmax/testing/distributed.py:122-179``): run a function on ``world_size`` ranks started
with ``multiprocessing`` spawn, each joining a process group on 127.0.0.1 with a free port (gloo on CPU; nccl when
``backend="nccl"`` and enough GPUs exist, otherwise the test is skipped).  Exceptions of any rank are re-raised in the
parent with the rank's traceback; a rank that hangs is killed after ``timeout`` seconds.
"""

from __future__ import annotations

import datetime
import io
import os
import socket
import sys
import traceback
from typing import Any, Callable, Optional, Tuple

import torch
import torch.multiprocessing as mp

__all__ = ["run_distributed_test", "find_free_port"]


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world_size: int, port: int, backend: str, fn: Callable, args: Tuple, kwargs: dict, queue) -> None:
    import torch.distributed as dist

    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world_size),
                       "LOCAL_WORLD_SIZE": str(world_size), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                       "OLMAX_SHARED_FS_DIRS": os.environ.get("TMPDIR", "/tmp")})
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = ""
        torch.set_num_threads(max(1, (os.cpu_count() or 2) // world_size))
        dist.init_process_group(backend=backend, init_method=f"tcp://127.0.0.1:{port}", world_size=world_size, rank=rank,
                                timeout=datetime.timedelta(seconds=120))
        from ..parallel import dist_utils

        dist_utils.init_distributed()  # attaches the host-side control group
        result = fn(*args, **kwargs)
        # tensors are serialised to bytes here: handing live tensors through a queue shares file descriptors that die
        # with this process
        buf = io.BytesIO()
        torch.save(result, buf)
        queue.put((rank, "ok", buf.getvalue()))
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
        raise


def run_distributed_test(fn: Callable, world_size: int = 2, backend: str = "gloo", func_args: Tuple = (),
                         func_kwargs: Optional[dict] = None, timeout: float = 180.0) -> list:
    """Run ``fn(*func_args, **func_kwargs)`` on every rank; returns the per-rank return values (picklable)."""
    if backend == "nccl":
        import pytest

        if not torch.cuda.is_available() or torch.cuda.device_count() < world_size:
            pytest.skip(f"needs {world_size} GPUs")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = find_free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, backend, fn, func_args, func_kwargs or {}, queue),
                         daemon=True) for r in range(world_size)]
    for p in procs:
        p.start()
    results: dict = {}
    errors = []
    import queue as pyqueue
    import time

    deadline = time.monotonic() + timeout
    while len(results) + len(errors) < world_size:
        remaining = deadline - time.monotonic()
        if remaining <= 0:
            break
        try:
            rank, status, payload = queue.get(timeout=min(remaining, 1.0))
        except pyqueue.Empty:
            if any(p.exitcode not in (None, 0) for p in procs) and queue.empty():
                break
            continue
        if status == "ok":
            results[rank] = torch.load(io.BytesIO(payload), weights_only=False)
        else:
            errors.append((rank, payload))
            break
    for p in procs:
        p.join(timeout=5 if not errors else 1)
        if p.is_alive():
            p.terminate()
    if errors:
        rank, tb = errors[0]
        raise RuntimeError(f"rank {rank} failed:\n{tb}")
    if len(results) < world_size:
        raise TimeoutError(f"only {len(results)} of {world_size} ranks finished within {timeout}s")
    return [results[r] for r in range(world_size)]

"""
Checkpoint save / restore of tensor trees and of sharded model + optimizer state
(role of ``olmax/checkpoint/utils.py:16-221``).

Layout of a checkpoint item (a directory)::

    <item>/_METADATA           JSON: {"arrays": {key: {"shape", "dtype"}}, "scalars": {key: value}}
    <item>/<key>/zarr.json     one zarr v3 array per tensor, stored in its GLOBAL logical shape
    <item>/<key>/c/i/j         one chunk per shard, written by the rank that owns it

Arrays are saved by global shape and restored by reading whatever region the target sharding needs, so a checkpoint
written under one mesh (say FSDP-8) restores under another (HSDP 2x4, a single GPU, ...).  Saving can run in the
background: tensors are first copied to host memory, then a thread writes the files (at most one save in flight).
"""

from __future__ import annotations

import concurrent.futures
import json
import logging
import os
import threading
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import fs
from ..parallel import dist_utils
from ..parallel.param_store import ParamStore
from ..types import PathOrStr
from ..utils.tree import tree_flatten_with_paths
from . import zarr3

__all__ = ["AsyncSaveHandle", "save", "restore", "get_metadata", "restore_from_metadata", "save_sharded",
           "restore_sharded", "write_json", "read_json"]

log = logging.getLogger(__name__)
METADATA = "_METADATA"


class AsyncSaveHandle:
    """Returned by a non-blocking save; ``wait()`` joins the writer thread and re-raises its error."""

    def __init__(self, thread: Optional[threading.Thread] = None, on_done: Optional[Callable[[], None]] = None):
        self._thread = thread
        self._error: Optional[BaseException] = None
        self._on_done = on_done
        self._finished = thread is None

    def _run(self, fn: Callable[[], None]) -> None:
        try:
            fn()
        except BaseException as e:  # noqa: BLE001 - re-raised in wait()
            self._error = e

    def done(self) -> bool:
        return self._thread is None or not self._thread.is_alive()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err
        if not self._finished:
            self._finished = True
            if self._on_done is not None:
                self._on_done()


def write_json(path: Path, obj: Any) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    tmp.write_text(json.dumps(obj, indent=1, sort_keys=True))
    os.replace(tmp, path)


def read_json(path: Path) -> Any:
    return json.loads(Path(path).read_text())


def _split_tree(tree: Any) -> Tuple[Dict[str, torch.Tensor], Dict[str, Any]]:
    arrays: Dict[str, torch.Tensor] = {}
    scalars: Dict[str, Any] = {}

    def visit(node: Any, prefix: str) -> None:
        if isinstance(node, torch.Tensor):
            arrays[prefix] = node
        elif isinstance(node, dict):
            for k, v in node.items():
                visit(v, f"{prefix}.{k}" if prefix else str(k))
        elif isinstance(node, (list, tuple)):
            for i, v in enumerate(node):
                visit(v, f"{prefix}.{i}" if prefix else str(i))
        else:
            scalars[prefix] = node

    visit(tree, "")
    return arrays, scalars


def _unflatten(flat: Dict[str, Any]) -> Any:
    root: Dict[str, Any] = {}
    for key, value in flat.items():
        if key == "":
            return value
        node = root
        parts = key.split(".")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = value
    return root


def save(directory: PathOrStr, tree: Any, block: bool = True, force: bool = False) -> AsyncSaveHandle:
    """
    Save a tree (nested dicts / lists of tensors and JSON-able leaves) of REPLICATED values: file-system rank 0 writes,
    everyone else returns immediately.  ``force`` overwrites an existing non-empty directory.
    """
    target = Path(fs.normalize_path(directory))
    if not force and target.exists() and any(target.iterdir()):
        raise FileExistsError(f"checkpoint directory {target} is not empty (pass force=True to overwrite)")
    if dist_utils.get_process_filesystem_rank() != 0:
        return AsyncSaveHandle()
    arrays, scalars = _split_tree(tree)
    host = {k: v.detach().to("cpu", copy=True) for k, v in arrays.items()}

    def write() -> None:
        target.mkdir(parents=True, exist_ok=True)
        meta = {"arrays": {}, "scalars": scalars, "tree_keys": sorted(list(host) + list(scalars))}
        for key, t in host.items():
            adir = target / (key or "_root")
            zarr3.write_metadata(adir, t.shape, t.shape if t.dim() else (), t.dtype)
            zarr3.write_chunk(adir, [0] * t.dim(), t)
            meta["arrays"][key] = {"shape": list(t.shape), "dtype": zarr3.TORCH_TO_ZARR[t.dtype]}
        write_json(target / METADATA, meta)

    if block:
        write()
        return AsyncSaveHandle()
    handle = AsyncSaveHandle.__new__(AsyncSaveHandle)
    AsyncSaveHandle.__init__(handle, None)
    th = threading.Thread(target=lambda: handle._run(write), name="checkpoint-writer", daemon=True)
    handle._thread, handle._finished = th, False
    th.start()
    return handle


def get_metadata(directory: PathOrStr) -> Dict[str, Any]:
    return read_json(Path(fs.normalize_path(directory)) / METADATA)


def restore_from_metadata(directory: PathOrStr, device: Optional[torch.device] = None) -> Any:
    """Rebuild the saved tree without a template (dict-of-dicts keyed by the saved paths)."""
    d = Path(fs.normalize_path(directory))
    meta = get_metadata(d)
    flat: Dict[str, Any] = dict(meta.get("scalars", {}))
    for key in meta["arrays"]:
        t = zarr3.read_full(d / (key or "_root"))
        flat[key] = t.to(device) if device is not None else t
    return _unflatten(flat)


def restore(directory: PathOrStr, target: Any) -> Any:
    """Restore into the structure of ``target``: tensors are read into the target leaf's dtype and device."""
    d = Path(fs.normalize_path(directory))
    meta = get_metadata(d)

    def visit(node: Any, prefix: str) -> Any:
        if isinstance(node, torch.Tensor):
            if prefix not in meta["arrays"]:
                raise KeyError(f"checkpoint {d} has no array '{prefix}'")
            t = zarr3.read_full(d / (prefix or "_root"))
            if tuple(t.shape) != tuple(node.shape):
                raise ValueError(f"'{prefix}': checkpoint shape {tuple(t.shape)} != target shape {tuple(node.shape)}")
            return t.to(device=node.device, dtype=node.dtype)
        if isinstance(node, dict):
            return {k: visit(v, f"{prefix}.{k}" if prefix else str(k)) for k, v in node.items()}
        if isinstance(node, (list, tuple)):
            return type(node)(visit(v, f"{prefix}.{i}" if prefix else str(i)) for i, v in enumerate(node))
        return meta.get("scalars", {}).get(prefix, node)

    return visit(target, "")


# ----------------------------------------------------------------------------------------------------------------------
# sharded state (ParamStore-shaped flat buffers)
# ----------------------------------------------------------------------------------------------------------------------
def _owns_chunk(store: ParamStore, meta) -> bool:
    """Exactly one rank writes each chunk: replicate coordinate 0, and TP coordinate 0 for TP-replicated params."""
    mesh = store.mesh
    if mesh.replicate.rank != 0:
        return False
    if meta.tp_dim is None and mesh.tp.rank != 0:
        return False
    return True


def _chunk_index(store: ParamStore, meta) -> List[int]:
    idx = [0] * len(meta.shape)
    tp, sh = store.mesh.tp, store.mesh.shard
    if meta.tp_dim is not None and tp.size > 1:
        idx[meta.tp_dim] = tp.rank
    if meta.tp_dim == 0 and tp.size > 1:
        idx[0] = tp.rank * sh.size + sh.rank
    else:
        idx[0] = sh.rank
    return idx


def save_sharded(directory: PathOrStr, store: ParamStore, buffers: Dict[str, torch.Tensor],
                 scalars: Optional[Dict[str, Any]] = None, block: bool = True) -> AsyncSaveHandle:
    """
    Save flat buffers laid out like ``store.master`` (``{"": master}`` for parameters, ``{"mu": ..., "nu": ...}`` for
    optimizer moments) as global-shape arrays named ``<prefix>.<param name>``.  Every rank writes the chunks it owns.
    The caller is responsible for barriers around the save (see ``SimpleCheckpointer``).
    """
    target = Path(fs.normalize_path(directory))
    work: List[Tuple[str, Any, List[int], torch.Tensor]] = []
    meta_out = {"arrays": {}, "scalars": scalars or {}}
    for prefix, flat in buffers.items():
        for m in store.metas:
            key = f"{prefix}.{m.name}" if prefix else m.name
            meta_out["arrays"][key] = {"shape": list(m.shape), "dtype": zarr3.TORCH_TO_ZARR[flat.dtype],
                                       "chunk_shape": list(m.local_shape)}
            if _owns_chunk(store, m):
                local = flat[m.offset : m.offset + m.numel_local].view(m.local_shape)
                work.append((key, m, _chunk_index(store, m), local.detach().to("cpu", copy=True)))
    is_writer0 = dist_utils.get_rank() == 0

    def write() -> None:
        target.mkdir(parents=True, exist_ok=True)
        for key, m, idx, t in work:
            if all(i == 0 for i in idx):
                zarr3.write_metadata(target / key, m.shape, m.local_shape, t.dtype)
        # all of this rank's chunks at once: a native thread pool writes them in parallel (checksummed, atomic renames)
        zarr3.write_chunks([(target / key, idx, t) for key, m, idx, t in work])
        if is_writer0:
            write_json(target / METADATA, meta_out)

    if block:
        write()
        return AsyncSaveHandle()
    handle = AsyncSaveHandle(None)
    th = threading.Thread(target=lambda: handle._run(write), name="checkpoint-writer", daemon=True)
    handle._thread, handle._finished = th, False
    th.start()
    return handle


def restore_sharded(directory: PathOrStr, store: ParamStore, buffers: Dict[str, torch.Tensor]) -> Dict[str, Any]:
    """Inverse of :func:`save_sharded` under ANY mesh: each rank reads the region of each array that its shard covers.
    Returns the saved scalars."""
    d = Path(fs.normalize_path(directory))
    meta = get_metadata(d)
    tp, sh = store.mesh.tp, store.mesh.shard
    jobs = []
    for prefix, flat in buffers.items():
        for m in store.metas:
            key = f"{prefix}.{m.name}" if prefix else m.name
            if key not in meta["arrays"]:
                raise KeyError(f"checkpoint {d} has no array '{key}'")
            if tuple(meta["arrays"][key]["shape"]) != tuple(m.shape):
                raise ValueError(f"'{key}': checkpoint shape {meta['arrays'][key]['shape']} != model shape {list(m.shape)}")
            start = [0] * len(m.shape)
            if m.tp_dim is not None and tp.size > 1:
                start[m.tp_dim] = tp.rank * m.tp_shape[m.tp_dim]
            start[0] += sh.rank * m.local_shape[0]
            jobs.append((key, start, m, flat))

    def read(job):
        key, start, m, _flat = job
        return zarr3.read_region(d / key, start, m.local_shape)

    # the chunk reads (native code: file I/O + checksum, outside the interpreter lock) run on a few threads; the copies
    # into the flat buffers stay on this thread, in order
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for job, region in zip(jobs, pool.map(read, jobs)):
            _key, _start, m, flat = job
            dst = flat[m.offset : m.offset + m.numel_local].view(m.local_shape)
            dst.copy_(region.to(dst.dtype))
    return meta.get("scalars", {})

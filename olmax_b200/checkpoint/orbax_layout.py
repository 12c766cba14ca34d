"""
The checkpoint layout Orbax produces for the reference (``olmax/checkpoint/utils.py:153-159``: an
``AsyncCheckpointer(PyTreeCheckpointHandler(use_ocdbt=True, use_zarr3=True))``; ``olmax/train/checkpointer.py:98-123``:
a composite of such items plus a JSON item), written and read without Orbax or TensorStore::

    <step dir>/_CHECKPOINT_METADATA          JSON: item handlers, timestamps
    <step dir>/trainer/metadata              JSON item (step, epoch, tokens seen)
    <step dir>/<item>/_METADATA              JSON: the item's tree (one entry per leaf: key path and value type)
    <step dir>/<item>/_sharding              JSON: per array, the named sharding it was saved with
    <step dir>/<item>/manifest.ocdbt         OCDBT database merged over the processes ...
    <step dir>/<item>/d/<hex>                ... its B+tree nodes
    <step dir>/<item>/ocdbt.process_<i>/     the database process i wrote: manifest.ocdbt + d/<hex> (chunk payloads)

Inside the database every array leaf ``a.b.c`` is a zarr v3 array: key ``a.b.c/zarr.json`` (metadata) and one key per
chunk ``a.b.c/c/<i>/<j>`` (``a.b.c/c`` for a scalar).  An array is stored in its GLOBAL shape with one chunk per
shard, written by the process that owns the shard; a reader assembles whatever region its own sharding needs, so a
checkpoint restores under a different mesh.

Tree naming follows the reference's objects so that items line up with the ones OLMax writes: parameters by module
path (``layers.0.attention.q_proj.weight``; the reference's scan mode stacks all layers as ``layers.0.*`` with a
leading ``[num_layers]`` dimension, which :func:`restore_store_item` also accepts), and the optimizer state as the optax
tree of ``olmax/optim/config.py:125-156``: ``MultiSteps(inject_hyperparams(adamw))`` =
``{mini_step, gradient_step, inner_opt_state: {count, hyperparams, hyperparams_states, inner_state: [ScaleByAdamState
{count, mu, nu}, ...]}, acc_grads}`` (without the ``inner_opt_state`` level for one micro-batch, and nested under tuple
index ``1`` behind a ``0.global_norm`` when gradients are clipped).

Limits, stated plainly: the byte formats are implemented from their published descriptions and verified by round trip
and hand-built fixtures here, not against Orbax / TensorStore (neither is installable offline), and ``_sharding`` /
``_METADATA`` carry the fields those descriptions name, not necessarily every field a given Orbax version emits.
"""

from __future__ import annotations

import base64
import json
import math
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parallel import dist_utils
from ..parallel.param_store import ParamStore
from . import zarr3
from .ocdbt import OcdbtReader, OcdbtWriter, merge_process_databases

__all__ = ["OCDBT_FORMAT", "array_metadata", "write_array", "ItemWriter", "finalize_item", "ItemReader",
           "save_store_item", "restore_store_item", "optax_prefixes", "write_checkpoint_metadata", "tree_metadata_entry"]

OCDBT_FORMAT = "ocdbt"
_NP = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "int64": np.int64, "int32": np.int32,
       "int16": np.int16, "int8": np.int8, "uint8": np.uint8, "bool": np.bool_, "bfloat16": np.uint16}


# ----------------------------------------------------------------------------------------------------------------------
# zarr v3 arrays inside a key-value store
# ----------------------------------------------------------------------------------------------------------------------
def array_metadata(shape: Sequence[int], chunk_shape: Sequence[int], dtype: torch.dtype) -> bytes:
    """``zarr.json`` of a regular-grid array: default chunk keys (``c/i/j``), little-endian ``bytes`` codec."""
    fill: Any = False if dtype == torch.bool else (0 if not dtype.is_floating_point else 0.0)
    return json.dumps({
        "zarr_format": 3, "node_type": "array", "shape": [int(s) for s in shape], "data_type": zarr3.TORCH_TO_ZARR[dtype],
        "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [int(s) for s in chunk_shape]}},
        "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
        "fill_value": fill, "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}], "attributes": {},
    }, sort_keys=True).encode()


def chunk_key(name: str, index: Sequence[int]) -> str:
    return f"{name}/c" + "".join(f"/{int(i)}" for i in index)


def _tensor_bytes(t: torch.Tensor) -> memoryview:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return memoryview(t.numpy()).cast("B") if t.numel() else memoryview(b"")


def write_array(writer: OcdbtWriter, name: str, t: torch.Tensor) -> None:
    """A whole (replicated) array as a single chunk."""
    writer.put(f"{name}/zarr.json", array_metadata(t.shape, t.shape, t.dtype))
    writer.put(chunk_key(name, [0] * t.dim()), _tensor_bytes(t))


def tree_metadata_entry(path: Sequence[str], value_type: str = "jax.Array") -> Tuple[str, dict]:
    """(key, value) of one leaf in ``_METADATA``'s ``tree_metadata``: the key is the Python repr of the key tuple;
    key_type 1 marks a sequence index, 2 a dictionary / attribute name."""
    keys = [{"key": p, "key_type": 1 if p.isdigit() else 2} for p in path]
    return str(tuple(path)), {"key_metadata": keys, "value_metadata": {"value_type": value_type, "skip_deserialize": False}}


class ItemWriter:
    """One process's share of one PyTree item: ``<item>/ocdbt.process_<rank>/``."""

    def __init__(self, item_dir: Path, process_index: int):
        self.item_dir = Path(item_dir)
        self.process_index = process_index
        self.db = OcdbtWriter(self.item_dir / f"ocdbt.process_{process_index}")

    def commit(self) -> None:
        self.db.commit()


def finalize_item(item_dir: Path, n_processes: int, leaves: Dict[str, dict], sharding: Optional[Dict[str, dict]] = None) -> None:
    """Run by ONE process after every process has committed: merge the per-process databases into the item's
    top-level ``manifest.ocdbt`` and write ``_METADATA`` (``leaves``: dotted leaf name -> {"value_type", "shape",
    "dtype"}) and ``_sharding``."""
    item_dir = Path(item_dir)
    merge_process_databases(item_dir, [f"ocdbt.process_{i}" for i in range(n_processes)])
    tree = {}
    for name, info in leaves.items():
        k, v = tree_metadata_entry(name.split("."), info.get("value_type", "jax.Array"))
        for extra in ("shape", "dtype", "write_shape"):
            if extra in info:
                v["value_metadata"][extra] = info[extra]
        tree[k] = v
    (item_dir / "_METADATA").write_text(json.dumps({"tree_metadata": tree, "use_zarr3": True,
                                                    "store_array_data_equal_to_fill_value": True, "custom_metadata": None},
                                                   indent=1))
    if sharding:
        enc = {base64.b64encode(n.encode()).decode(): json.dumps(s) for n, s in sharding.items()}
        (item_dir / "_sharding").write_text(json.dumps(enc, indent=1))


class ItemReader:
    """Arrays of one PyTree item, read through the merged database (or the process databases when the merged manifest
    is missing)."""

    def __init__(self, item_dir: Path):
        self.item_dir = Path(item_dir)
        self.db = OcdbtReader(self.item_dir)
        self._meta: Dict[str, dict] = {}

    def close(self) -> None:
        self.db.close()

    def array_names(self) -> List[str]:
        return sorted(k[: -len("/zarr.json")] for k in self.db.keys() if k.endswith("/zarr.json"))

    def meta(self, name: str) -> dict:
        if name not in self._meta:
            m = json.loads(self.db.get(f"{name}/zarr.json"))
            if m.get("zarr_format") != 3 or m.get("node_type") != "array":
                raise ValueError(f"{name}: not a zarr v3 array")
            codecs = [c["name"] for c in m.get("codecs", [])]
            if not codecs or codecs[0] != "bytes" or any(c not in ("bytes", "zstd", "crc32c") for c in codecs):
                raise ValueError(f"{name}: unsupported codec chain {codecs}")
            if m["codecs"][0].get("configuration", {}).get("endian", "little") != "little":
                raise ValueError(f"{name}: big-endian arrays are not supported")
            self._meta[name] = m
        return self._meta[name]

    def _chunk(self, name: str, m: dict, index: Sequence[int]) -> Optional[np.ndarray]:
        key = chunk_key(name, index)
        if key not in self.db:
            return None   # a missing chunk holds the fill value
        raw = self.db.get(key)
        for c in reversed(m["codecs"][1:]):
            if c["name"] == "crc32c":
                if int.from_bytes(raw[-4:], "little") != zarr3.crc32c(raw[:-4]):
                    raise ValueError(f"{key}: CRC-32C mismatch")
                raw = raw[:-4]
            elif c["name"] == "zstd":
                from .ocdbt import zstd_decompress
                raw = zstd_decompress(raw)
        cs = m["chunk_grid"]["configuration"]["chunk_shape"]
        arr = np.frombuffer(raw, dtype=_NP[m["data_type"]])
        if arr.size != int(math.prod(cs)):
            raise ValueError(f"{key}: {arr.size} elements, chunk shape {cs}")
        return arr.reshape(cs)

    def read_region(self, name: str, start: Sequence[int], shape: Sequence[int]) -> torch.Tensor:
        m = self.meta(name)
        full, cs = m["shape"], m["chunk_grid"]["configuration"]["chunk_shape"]
        nd = len(full)
        if len(start) != nd or any(start[d] < 0 or start[d] + shape[d] > full[d] for d in range(nd)):
            raise ValueError(f"{name}: region {list(start)}+{list(shape)} outside the array {full}")
        out = np.full(tuple(shape), m.get("fill_value", 0) or 0, dtype=_NP[m["data_type"]])
        lo = [start[d] // cs[d] for d in range(nd)]
        hi = [(start[d] + shape[d] - 1) // cs[d] if shape[d] else lo[d] - 1 for d in range(nd)]
        for idx in np.ndindex(*[max(0, hi[d] - lo[d] + 1) for d in range(nd)]) if nd else [()]:
            cidx = [lo[d] + idx[d] for d in range(nd)]
            chunk = self._chunk(name, m, cidx)
            if chunk is None:
                continue
            src, dst = [], []
            for d in range(nd):
                c0 = cidx[d] * cs[d]
                a, b = max(start[d], c0), min(start[d] + shape[d], c0 + cs[d], full[d])
                src.append(slice(a - c0, b - c0))
                dst.append(slice(a - start[d], b - start[d]))
            out[tuple(dst)] = chunk[tuple(src)]
        t = torch.from_numpy(out)
        return t.view(torch.bfloat16) if m["data_type"] == "bfloat16" else t

    def read(self, name: str) -> torch.Tensor:
        m = self.meta(name)
        return self.read_region(name, [0] * len(m["shape"]), m["shape"])


# ----------------------------------------------------------------------------------------------------------------------
# ParamStore-shaped state
# ----------------------------------------------------------------------------------------------------------------------
def optax_prefixes(num_microbatches: int, clipped: bool) -> Tuple[str, str]:
    """(prefix of the MultiSteps level or "", prefix of the InjectStatefulHyperparamsState) in the optax tree."""
    outer = "inner_opt_state." if num_microbatches > 1 else ""
    return outer, outer + ("1." if clipped else "")


def _named_sharding(store: ParamStore, meta) -> dict:
    """The reference's placement of a parameter as a JSON named sharding: dim 0 over the shard axis, the TP dim over
    the TP axis (``olmax/distributed/parallel.py:309-334``)."""
    mesh = store.mesh
    axes, shape = [], []
    for name, g in (("fsdp_replicate", mesh.replicate), ("fsdp_shard", mesh.shard), ("tp", mesh.tp), ("cp", mesh.cp)):
        if g.size > 1 or name == "fsdp_shard":
            axes.append(name)
            shape.append(g.size)
    spec: List[Any] = [None] * len(meta.shape)
    if meta.tp_dim is not None and mesh.tp.size > 1:
        spec[meta.tp_dim] = "tp"
    spec[0] = "fsdp_shard" if spec[0] is None else ["tp", "fsdp_shard"]
    return {"sharding_type": "NamedSharding", "shape": shape, "axis_names": axes, "partition_spec": spec}


def save_store_item(item_dir: Path, store: ParamStore, buffers: Dict[str, torch.Tensor],
                    scalars: Optional[Dict[str, Any]] = None, zero_arrays: Sequence[str] = ()) -> Tuple[Dict[str, dict], Dict[str, dict]]:
    """This process's part of an item holding flat buffers laid out like ``store.master`` (``{"": master}`` or
    ``{"inner_state.0.mu": exp_avg, ...}``), 0-d ``scalars`` and, for every prefix in ``zero_arrays``, parameter-shaped
    arrays that are all zero (metadata only: a chunk that is absent holds the fill value).  Every process calls this and
    then a barrier; one process then calls :func:`finalize_item` with the returned (leaves, sharding)."""
    from .utils import _chunk_index, _owns_chunk

    rank = dist_utils.get_rank()
    w = ItemWriter(item_dir, rank)
    leaves: Dict[str, dict] = {}
    sharding: Dict[str, dict] = {}
    for prefix, flat in buffers.items():
        for m in store.metas:
            key = f"{prefix}.{m.name}" if prefix else m.name
            leaves[key] = {"shape": list(m.shape), "dtype": zarr3.TORCH_TO_ZARR[flat.dtype], "write_shape": list(m.local_shape)}
            sharding[key] = _named_sharding(store, m)
            if not _owns_chunk(store, m):
                continue
            idx = _chunk_index(store, m)
            if all(i == 0 for i in idx):
                w.db.put(f"{key}/zarr.json", array_metadata(m.shape, m.local_shape, flat.dtype))
            w.db.put(chunk_key(key, idx), _tensor_bytes(flat[m.offset : m.offset + m.numel_local].view(m.local_shape)))
    for prefix in zero_arrays:
        for m in store.metas:
            key = f"{prefix}.{m.name}"
            leaves[key] = {"shape": list(m.shape), "dtype": "float32", "write_shape": list(m.local_shape)}
            sharding[key] = _named_sharding(store, m)
            if rank == 0:
                w.db.put(f"{key}/zarr.json", array_metadata(m.shape, m.local_shape, torch.float32))
    for name, value in (scalars or {}).items():
        t = value if isinstance(value, torch.Tensor) else torch.tensor(value)
        if t.dtype == torch.int64 and not isinstance(value, torch.Tensor):
            t = t.to(torch.int32)      # optax counters are int32
        if t.dtype == torch.float64:
            t = t.to(torch.float32)
        leaves[name] = {"shape": [], "dtype": zarr3.TORCH_TO_ZARR[t.dtype]}
        if rank == 0:
            write_array(w.db, name, t.reshape(()))
    w.commit()
    return leaves, sharding


def restore_store_item(item_dir: Path, store: ParamStore, buffers: Dict[str, torch.Tensor],
                       scalar_names: Iterable[str] = (), single_replica: Optional[bool] = None) -> Dict[str, Any]:
    """Inverse of :func:`save_store_item` under ANY mesh; returns the requested scalars that exist.  A parameter
    ``layers.<i>.<rest>`` that is missing is looked up as row ``i`` of a stacked ``layers.0.<rest>`` array with a
    leading layer dimension (the reference's scan mode).

    ``single_replica`` (default: on whenever the mesh has more than one replica, like
    ``enable_single_replica_restoring`` of ``olmax/checkpoint/utils.py:169-221``): only the ranks of replica 0 read
    the files; every other replica receives its shards by a broadcast over the replicate group, so the file system
    serves each byte once however many replicas there are."""
    rep = store.mesh.replicate
    if single_replica is None:
        single_replica = rep.size > 1
    if single_replica and rep.size > 1:
        import torch.distributed as dist

        scalars: Dict[str, Any] = {}
        if rep.rank == 0:
            scalars = restore_store_item(item_dir, store, buffers, scalar_names, single_replica=False)
        src = rep.ranks[0]
        for flat in buffers.values():
            dist.broadcast(flat, src=src, group=rep.pg)
        box = [scalars]
        dist.broadcast_object_list(box, src=src, group=rep.pg)
        return box[0]
    r = ItemReader(item_dir)
    try:
        names = set(r.array_names())
        tp, sh = store.mesh.tp, store.mesh.shard
        n_layers = len({m.name.split(".")[1] for m in store.metas if m.name.startswith("layers.")})
        for prefix, flat in buffers.items():
            for m in store.metas:
                key = f"{prefix}.{m.name}" if prefix else m.name
                start = [0] * len(m.shape)
                if m.tp_dim is not None and tp.size > 1:
                    start[m.tp_dim] = tp.rank * m.tp_shape[m.tp_dim]
                start[0] += sh.rank * m.local_shape[0]
                dst = flat[m.offset : m.offset + m.numel_local].view(m.local_shape)
                if key in names and tuple(r.meta(key)["shape"]) == tuple(m.shape):
                    dst.copy_(r.read_region(key, start, m.local_shape).to(dst.dtype))
                    continue
                parts = m.name.split(".")
                stacked = ".".join(([prefix] if prefix else []) + ["layers", "0"] + parts[2:])
                if (parts[0] == "layers" and stacked in names
                        and tuple(r.meta(stacked)["shape"]) == (n_layers,) + tuple(m.shape)):
                    region = r.read_region(stacked, [int(parts[1])] + start, [1] + list(m.local_shape))
                    dst.copy_(region[0].to(dst.dtype))
                    continue
                if key in names:
                    raise ValueError(f"'{key}': checkpoint shape {r.meta(key)['shape']} != model shape {list(m.shape)}")
                raise KeyError(f"checkpoint item {item_dir} has no array '{key}'")
        out = {}
        for name in scalar_names:
            if name in names:
                out[name] = r.read(name).item()
        return out
    finally:
        r.close()


def write_checkpoint_metadata(step_dir: Path, pytree_items: Sequence[str], json_items: Sequence[str], started_ns: int) -> None:
    """``_CHECKPOINT_METADATA`` of a composite checkpoint: written last, its presence marks the step as complete."""
    handlers = {name: "orbax.checkpoint._src.handlers.pytree_checkpoint_handler.PyTreeCheckpointHandler" for name in pytree_items}
    handlers.update({name: "orbax.checkpoint._src.handlers.json_checkpoint_handler.JsonCheckpointHandler" for name in json_items})
    meta = {"item_handlers": handlers, "metrics": {}, "performance_metrics": {}, "init_timestamp_nsecs": int(started_ns),
            "commit_timestamp_nsecs": time.time_ns(), "custom_metadata": {"format": OCDBT_FORMAT, "writer": "olmax_b200"}}
    tmp = Path(step_dir) / "_CHECKPOINT_METADATA.tmp"
    tmp.write_text(json.dumps(meta, indent=1))
    tmp.replace(Path(step_dir) / "_CHECKPOINT_METADATA")

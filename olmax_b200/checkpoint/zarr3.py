"""
Minimal zarr v3 directory-store writer / reader for regular chunk grids.

An array lives in its own directory: ``zarr.json`` (zarr v3 array metadata: shape, data_type, regular chunk grid,
default chunk-key encoding ``c/i/j``, a single ``bytes`` little-endian codec) plus one file per chunk.  A parameter
sharded over ranks is exactly such a grid (chunk = one rank's shard), so every rank writes its own chunk files without
gathering, and a reader can assemble any hyper-rectangle, which is what makes restoring under a different sharding
possible.  The reference stores zarr v3 arrays too, but packed inside an OCDBT key-value database by TensorStore
(``olmax/checkpoint/utils.py:153-159``); this module writes the same arrays as plain files.
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = ["write_metadata", "write_chunk", "read_metadata", "read_region", "read_full", "TORCH_TO_ZARR"]

TORCH_TO_ZARR = {
    torch.float32: "float32", torch.float64: "float64", torch.float16: "float16", torch.bfloat16: "bfloat16",
    torch.int64: "int64", torch.int32: "int32", torch.int16: "int16", torch.int8: "int8", torch.uint8: "uint8",
    torch.bool: "bool",
}
ZARR_TO_TORCH = {v: k for k, v in TORCH_TO_ZARR.items()}
_ITEMSIZE = {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2, "int64": 8, "int32": 4, "int16": 2, "int8": 1,
             "uint8": 1, "bool": 1}


def write_metadata(array_dir: Path, shape: Sequence[int], chunk_shape: Sequence[int], dtype: torch.dtype) -> None:
    array_dir.mkdir(parents=True, exist_ok=True)
    meta = {
        "zarr_format": 3,
        "node_type": "array",
        "shape": [int(s) for s in shape],
        "data_type": TORCH_TO_ZARR[dtype],
        "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [int(s) for s in chunk_shape] or [1]}},
        "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
        "fill_value": 0,
        "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}],
        "attributes": {},
    }
    tmp = array_dir / f"zarr.json.tmp{os.getpid()}"
    tmp.write_text(json.dumps(meta))
    os.replace(tmp, array_dir / "zarr.json")


def _chunk_path(array_dir: Path, index: Sequence[int]) -> Path:
    return array_dir / "c" / Path(*[str(int(i)) for i in index]) if len(index) else array_dir / "c"


def write_chunk(array_dir: Path, index: Sequence[int], data: torch.Tensor) -> None:
    """Write one chunk (a CPU tensor of exactly the chunk shape) atomically."""
    path = _chunk_path(array_dir, index)
    path.parent.mkdir(parents=True, exist_ok=True)
    t = data.detach().contiguous().cpu()
    raw = t.view(torch.uint8).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(tmp, "wb") as f:
        f.write(raw)
    os.replace(tmp, path)


def read_metadata(array_dir: Path) -> Dict:
    meta = json.loads((array_dir / "zarr.json").read_text())
    if meta.get("zarr_format") != 3 or meta.get("node_type") != "array":
        raise ValueError(f"{array_dir} is not a zarr v3 array")
    return meta


def _read_chunk(array_dir: Path, index: Sequence[int], chunk_shape: Sequence[int], dtype_name: str) -> torch.Tensor:
    path = _chunk_path(array_dir, index)
    n = int(np.prod(chunk_shape)) if len(chunk_shape) else 1
    if not path.exists():
        return torch.zeros(tuple(chunk_shape), dtype=ZARR_TO_TORCH[dtype_name])
    raw = path.read_bytes()
    expect = n * _ITEMSIZE[dtype_name]
    if len(raw) != expect:
        raise ValueError(f"chunk {path} has {len(raw)} bytes, expected {expect} (truncated or corrupt checkpoint)")
    buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    return buf.view(ZARR_TO_TORCH[dtype_name]).reshape(tuple(chunk_shape))


def read_region(array_dir: Path, start: Sequence[int], shape: Sequence[int]) -> torch.Tensor:
    """Assemble the hyper-rectangle ``[start, start + shape)`` from whichever chunks overlap it."""
    meta = read_metadata(array_dir)
    full_shape = meta["shape"]
    dtype_name = meta["data_type"]
    if len(full_shape) == 0:
        return _read_chunk(array_dir, (), (), dtype_name).reshape(())
    cshape = meta["chunk_grid"]["configuration"]["chunk_shape"]
    out = torch.zeros(tuple(shape), dtype=ZARR_TO_TORCH[dtype_name])
    ranges = []
    for d in range(len(full_shape)):
        lo, hi = start[d] // cshape[d], (start[d] + shape[d] - 1) // cshape[d]
        ranges.append(range(lo, hi + 1))
    import itertools

    for idx in itertools.product(*ranges):
        chunk = _read_chunk(array_dir, idx, cshape, dtype_name)
        src_sl, dst_sl = [], []
        for d, ci in enumerate(idx):
            c0 = ci * cshape[d]
            lo = max(c0, start[d])
            hi = min(c0 + cshape[d], start[d] + shape[d], full_shape[d])
            src_sl.append(slice(lo - c0, hi - c0))
            dst_sl.append(slice(lo - start[d], hi - start[d]))
        out[tuple(dst_sl)] = chunk[tuple(src_sl)]
    return out


def read_full(array_dir: Path) -> torch.Tensor:
    meta = read_metadata(array_dir)
    return read_region(array_dir, [0] * len(meta["shape"]), meta["shape"])

"""
Minimal zarr v3 directory-store writer / reader for regular chunk grids.

An array lives in its own directory: ``zarr.json`` (zarr v3 array metadata: shape, data_type, regular chunk grid,
default chunk-key encoding ``c/i/j``, the ``bytes`` little-endian codec followed by the ``crc32c`` checksum codec, i.e.
every chunk file ends in the 4-byte CRC-32C of its payload) plus one file per chunk.  Chunk files are written and read
by the native library ``lib/libolmax_ckpt.so`` (``csrc/ckpt_io.cpp``: a thread pool outside the interpreter lock,
atomic renames, checksum verification); when that library is missing (no C++ compiler) the same bytes are produced
in Python.  A parameter
sharded over ranks is exactly such a grid (chunk = one rank's shard), so every rank writes its own chunk files without
gathering, and a reader can assemble any hyper-rectangle, which is what makes restoring under a different sharding
possible.  The reference stores zarr v3 arrays too, but packed inside an OCDBT key-value database by TensorStore
(``olmax/checkpoint/utils.py:153-159``); this module writes the same arrays as plain files.
"""

from __future__ import annotations

import ctypes
import json
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = ["write_metadata", "write_chunk", "write_chunks", "read_metadata", "read_region", "read_full", "crc32c",
           "TORCH_TO_ZARR"]

TORCH_TO_ZARR = {
    torch.float32: "float32", torch.float64: "float64", torch.float16: "float16", torch.bfloat16: "bfloat16",
    torch.int64: "int64", torch.int32: "int32", torch.int16: "int16", torch.int8: "int8", torch.uint8: "uint8",
    torch.bool: "bool",
}
ZARR_TO_TORCH = {v: k for k, v in TORCH_TO_ZARR.items()}
_ITEMSIZE = {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2, "int64": 8, "int32": 4, "int16": 2, "int8": 1,
             "uint8": 1, "bool": 1}


# ---- native chunk I/O ------------------------------------------------------------------------------------------------
_NATIVE = None
_NATIVE_TRIED = False


def _native():
    """The checkpoint I/O library, built on first use when a C++ compiler exists; None otherwise."""
    global _NATIVE, _NATIVE_TRIED
    if _NATIVE_TRIED:
        return _NATIVE
    _NATIVE_TRIED = True
    if os.environ.get("OLMAX_B200_CKPT_NATIVE", "1") != "1":
        return None
    try:
        from ..csrc.build import build_host

        lib = ctypes.CDLL(str(build_host()))
        lib.ob_crc32c.restype = ctypes.c_uint32
        lib.ob_crc32c.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        sig = [ctypes.c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_void_p),
               ctypes.POINTER(ctypes.c_uint64), ctypes.c_int]
        lib.ob_ckpt_write_files.restype = ctypes.c_int
        lib.ob_ckpt_write_files.argtypes = sig + [ctypes.c_int, ctypes.c_int]
        lib.ob_ckpt_read_files.restype = ctypes.c_int
        lib.ob_ckpt_read_files.argtypes = sig + [ctypes.c_int]
        lib.ob_ckpt_last_error.restype = ctypes.c_char_p
        _NATIVE = lib
    except Exception:  # noqa: BLE001  (no compiler, read-only tree, ...)
        _NATIVE = None
    return _NATIVE


_CRC_TABLE: Optional[List[int]] = None


def crc32c(data: bytes) -> int:
    """CRC-32C (Castagnoli) of ``data``: native when the library is there, a table-driven loop otherwise."""
    lib = _native()
    if lib is not None:
        buf = (ctypes.c_char * len(data)).from_buffer_copy(data) if len(data) else None
        return int(lib.ob_crc32c(ctypes.cast(buf, ctypes.c_void_p) if buf is not None else None, len(data)))
    global _CRC_TABLE
    if _CRC_TABLE is None:
        table = []
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
            table.append(c)
        _CRC_TABLE = table
    crc = 0xFFFFFFFF
    for b in data:
        crc = (crc >> 8) ^ _CRC_TABLE[(crc ^ b) & 0xFF]
    return crc ^ 0xFFFFFFFF


def _as_bytes_tensor(data: torch.Tensor) -> torch.Tensor:
    t = data.detach().contiguous().cpu()
    return t.view(torch.uint8).reshape(-1) if t.dim() else t.reshape(1).view(torch.uint8)


def write_metadata(array_dir: Path, shape: Sequence[int], chunk_shape: Sequence[int], dtype: torch.dtype) -> None:
    array_dir.mkdir(parents=True, exist_ok=True)
    meta = {
        "zarr_format": 3,
        "node_type": "array",
        "shape": [int(s) for s in shape],
        "data_type": TORCH_TO_ZARR[dtype],
        "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [int(s) for s in chunk_shape]}},
        "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
        "fill_value": 0,
        "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "crc32c"}],
        "attributes": {},
    }
    tmp = array_dir / f"zarr.json.tmp{os.getpid()}"
    tmp.write_text(json.dumps(meta))
    os.replace(tmp, array_dir / "zarr.json")


def _chunk_path(array_dir: Path, index: Sequence[int]) -> Path:
    return array_dir / "c" / Path(*[str(int(i)) for i in index]) if len(index) else array_dir / "c"


def write_chunks(items: Sequence[Tuple[Path, Sequence[int], torch.Tensor]], n_threads: int = 8, fsync: bool = False) -> None:
    """Write many chunks ``(array_dir, chunk index, tensor of exactly the chunk shape)`` atomically, in parallel."""
    if not items:
        return
    paths, bufs = [], []
    for array_dir, index, data in items:
        path = _chunk_path(array_dir, index)
        path.parent.mkdir(parents=True, exist_ok=True)
        paths.append(path)
        bufs.append(_as_bytes_tensor(data))
    lib = _native()
    if lib is not None:
        n = len(items)
        c_paths = (ctypes.c_char_p * n)(*[str(p).encode() for p in paths])
        c_ptrs = (ctypes.c_void_p * n)(*[b.data_ptr() for b in bufs])
        c_sizes = (ctypes.c_uint64 * n)(*[b.numel() for b in bufs])
        rc = lib.ob_ckpt_write_files(n, c_paths, c_ptrs, c_sizes, 1, int(fsync), n_threads)
        if rc != 0:
            raise OSError(f"checkpoint write failed: {lib.ob_ckpt_last_error().decode()}")
        return
    for path, buf in zip(paths, bufs):
        raw = buf.numpy().tobytes()
        tmp = path.with_name(path.name + f".tmp{os.getpid()}")
        with open(tmp, "wb") as f:
            f.write(raw)
            f.write(crc32c(raw).to_bytes(4, "little"))
        os.replace(tmp, path)


def write_chunk(array_dir: Path, index: Sequence[int], data: torch.Tensor) -> None:
    """Write one chunk (a CPU tensor of exactly the chunk shape) atomically."""
    write_chunks([(array_dir, index, data)], n_threads=1)


def read_metadata(array_dir: Path) -> Dict:
    meta = json.loads((array_dir / "zarr.json").read_text())
    if meta.get("zarr_format") != 3 or meta.get("node_type") != "array":
        raise ValueError(f"{array_dir} is not a zarr v3 array")
    return meta


def _has_crc(meta: Dict) -> bool:
    return any(c.get("name") == "crc32c" for c in meta.get("codecs", []))


def _read_chunk(array_dir: Path, index: Sequence[int], chunk_shape: Sequence[int], dtype_name: str,
                has_crc: bool = False) -> torch.Tensor:
    path = _chunk_path(array_dir, index)
    n = int(np.prod(chunk_shape)) if len(chunk_shape) else 1
    if not path.exists():
        return torch.zeros(tuple(chunk_shape), dtype=ZARR_TO_TORCH[dtype_name])
    expect = n * _ITEMSIZE[dtype_name]
    lib = _native()
    if lib is not None:
        buf = torch.empty(expect, dtype=torch.uint8)
        c_paths = (ctypes.c_char_p * 1)(str(path).encode())
        c_ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
        c_sizes = (ctypes.c_uint64 * 1)(expect)
        if lib.ob_ckpt_read_files(1, c_paths, c_ptrs, c_sizes, int(has_crc), 1) != 0:
            raise ValueError(lib.ob_ckpt_last_error().decode())
    else:
        raw = path.read_bytes()
        if len(raw) != expect + (4 if has_crc else 0):
            raise ValueError(f"chunk {path} has {len(raw)} bytes, expected {expect + (4 if has_crc else 0)} "
                             f"(truncated or corrupt checkpoint)")
        if has_crc:
            raw, tail = raw[:expect], raw[expect:]
            if crc32c(raw) != int.from_bytes(tail, "little"):
                raise ValueError(f"chunk {path} checksum mismatch: corrupt checkpoint")
        buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    return buf.view(ZARR_TO_TORCH[dtype_name]).reshape(tuple(chunk_shape))


def _read_chunks(array_dir: Path, indices: Sequence[Sequence[int]], chunk_shape: Sequence[int], dtype_name: str,
                 has_crc: bool, n_threads: int = 8) -> List[torch.Tensor]:
    """Several chunks of one array; with the native library the files that exist are read by one threaded call."""
    lib = _native()
    if lib is None or len(indices) < 2:
        return [_read_chunk(array_dir, idx, chunk_shape, dtype_name, has_crc) for idx in indices]
    n_elems = int(np.prod(chunk_shape)) if len(chunk_shape) else 1
    expect = n_elems * _ITEMSIZE[dtype_name]
    out: List[Optional[torch.Tensor]] = [None] * len(indices)
    paths, bufs, slots = [], [], []
    for i, idx in enumerate(indices):
        path = _chunk_path(array_dir, idx)
        if not path.exists():     # a chunk that was never written reads as the fill value
            out[i] = torch.zeros(tuple(chunk_shape), dtype=ZARR_TO_TORCH[dtype_name])
            continue
        paths.append(str(path).encode())
        bufs.append(torch.empty(expect, dtype=torch.uint8))
        slots.append(i)
    if paths:
        n = len(paths)
        c_paths = (ctypes.c_char_p * n)(*paths)
        c_ptrs = (ctypes.c_void_p * n)(*[b.data_ptr() for b in bufs])
        c_sizes = (ctypes.c_uint64 * n)(*([expect] * n))
        if lib.ob_ckpt_read_files(n, c_paths, c_ptrs, c_sizes, int(has_crc), n_threads) != 0:
            raise ValueError(lib.ob_ckpt_last_error().decode())
        for i, buf in zip(slots, bufs):
            out[i] = buf.view(ZARR_TO_TORCH[dtype_name]).reshape(tuple(chunk_shape))
    return out  # type: ignore[return-value]


def read_region(array_dir: Path, start: Sequence[int], shape: Sequence[int]) -> torch.Tensor:
    """Assemble the hyper-rectangle ``[start, start + shape)`` from whichever chunks overlap it."""
    meta = read_metadata(array_dir)
    full_shape = meta["shape"]
    dtype_name = meta["data_type"]
    has_crc = _has_crc(meta)
    if len(full_shape) == 0:
        return _read_chunk(array_dir, (), (), dtype_name, has_crc).reshape(())
    cshape = meta["chunk_grid"]["configuration"]["chunk_shape"]
    out = torch.zeros(tuple(shape), dtype=ZARR_TO_TORCH[dtype_name])
    ranges = []
    for d in range(len(full_shape)):
        lo, hi = start[d] // cshape[d], (start[d] + shape[d] - 1) // cshape[d]
        ranges.append(range(lo, hi + 1))
    import itertools

    indices = list(itertools.product(*ranges))
    chunks = _read_chunks(array_dir, indices, cshape, dtype_name, has_crc)
    for idx, chunk in zip(indices, chunks):
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

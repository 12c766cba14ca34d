"""
In-tree build of the sm_100a kernel library.

Every ``.cu`` file beside this script is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an object
file under ``csrc/build/`` and the objects are linked into ``olmax_b200/lib/libolmax_b200.so``.  The library exposes a
plain C interface (``extern "C"``) that :mod:`olmax_b200.ops._lib` loads with :mod:`ctypes`, so the build needs neither
the PyTorch headers nor a GPU: nvcc cross-compiles on a CPU-only machine and the resulting ``.so`` is what runs on the
B200.

A second, host-only library, ``olmax_b200/lib/libolmax_ckpt.so`` (``ckpt_io.cpp``: threaded checkpoint chunk I/O with
CRC-32C), is compiled with g++ by :func:`build_host`.

Run as a script (``python -m olmax_b200.csrc.build``) or call :func:`build`.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List, Optional

CSRC = Path(__file__).resolve().parent
LIB_DIR = CSRC.parent / "lib"
LIB_PATH = LIB_DIR / "libolmax_b200.so"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=default",
]


def find_nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> List[Path]:
    return sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")))


def _fingerprint(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in _headers():
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    fp = _fingerprint(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == fp:
        return obj
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and res.stderr:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(fp)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and link the kernel library; returns its path."""
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.sha"):
            f.unlink()
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as pool:
        objs = list(pool.map(lambda s: _compile_one(nvcc, s, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        tmp = LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-Xcompiler", "-fPIC"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


CKPT_LIB_PATH = LIB_DIR / "libolmax_ckpt.so"


def build_host(force: bool = False) -> Path:
    """Compile the host-only checkpoint I/O library with the C++ compiler (no CUDA involved)."""
    src = CSRC / "ckpt_io.cpp"
    LIB_DIR.mkdir(exist_ok=True)
    if not force and CKPT_LIB_PATH.exists() and CKPT_LIB_PATH.stat().st_mtime >= src.stat().st_mtime:
        return CKPT_LIB_PATH
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found (set CXX)")
    tmp = CKPT_LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-msse4.2", str(src), "-o", str(tmp)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{cxx} failed for ckpt_io.cpp:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, CKPT_LIB_PATH)
    return CKPT_LIB_PATH


def is_stale() -> bool:
    """True when the library is missing or older than any source/header."""
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _sources() + _headers())


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_host(force="--force" in sys.argv))

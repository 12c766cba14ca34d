"""
Loader for the in-tree sm_100a kernel library (``olmax_b200/lib/libolmax_b200.so``).

The library has a plain C interface and is loaded with :mod:`ctypes`; tensors are passed as raw device pointers
together with the current CUDA stream.  On a machine with a GPU the library is mandatory: :func:`lib` raises if it
cannot be loaded, so a GPU run never falls back silently to PyTorch math.  On a CPU-only machine the ops in this
package use their PyTorch restatement instead (that path is what the gloo/CPU tests exercise).
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LOCK = threading.Lock()

# OLMAX_B200_LIB selects another build of the kernel library (e.g. one compiled with experimental -D switches)
LIB_PATH = Path(os.environ.get("OLMAX_B200_LIB") or (Path(__file__).resolve().parent.parent / "lib" / "libolmax_b200.so"))


class KernelError(RuntimeError):
    """Raised when a kernel launch is rejected by the host wrapper or a kernel reported an error status."""


class ObGemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p),
        ("lda", ctypes.c_longlong),
        ("b", ctypes.c_void_p),
        ("ldb", ctypes.c_longlong),
        ("b_shard_stride", ctypes.c_longlong),
        ("b2", ctypes.c_void_p),
        ("c", ctypes.c_void_p),
        ("ldc", ctypes.c_longlong),
        ("c2", ctypes.c_void_p),
        ("c3", ctypes.c_void_p),
        ("c_shards", ctypes.c_void_p),
        ("c_shard_stride", ctypes.c_longlong),
        ("M", ctypes.c_int),
        ("N", ctypes.c_int),
        ("Kc", ctypes.c_int),
        ("M_s", ctypes.c_int),
        ("N_s", ctypes.c_int),
        ("Kc_s", ctypes.c_int),
        ("a_mn", ctypes.c_int),
        ("b_mn", ctypes.c_int),
        ("epi", ctypes.c_int),
        ("alpha", ctypes.c_float),
        ("status", ctypes.c_void_p),
        ("max_ctas", ctypes.c_int),
        ("ag_src", ctypes.c_void_p),
        ("ag_src2", ctypes.c_void_p),
        ("ag_flags", ctypes.c_void_p),
        ("ag_rank", ctypes.c_int),
        ("pf_src", ctypes.c_void_p),
        ("pf_dst", ctypes.c_void_p),
        ("pf_dst_stride", ctypes.c_longlong),
        ("pf_off", ctypes.c_longlong),
        ("pf_bytes", ctypes.c_longlong),
        ("pf_shards", ctypes.c_int),
        ("pf_rank", ctypes.c_int),
        ("m_shard_rot", ctypes.c_int),
        ("group_m", ctypes.c_int),
        ("multi_box_mn", ctypes.c_int),
        ("no_tma_epilogue", ctypes.c_int),
        ("ag_on_a", ctypes.c_int),
        ("no_split_k", ctypes.c_int),
    ]


def _declare(lib: ctypes.CDLL) -> None:
    lib.ob_last_error.restype = ctypes.c_char_p
    lib.ob_gemm_bf16.restype = ctypes.c_int
    lib.ob_gemm_bf16.argtypes = [ctypes.POINTER(ObGemmArgs), ctypes.c_void_p]
    for name in ("ob_flash_attn_fwd", "ob_flash_attn_bwd"):
        if hasattr(lib, name):
            getattr(lib, name).restype = ctypes.c_int
            getattr(lib, name).argtypes = [ctypes.POINTER(ObAttnArgs), ctypes.c_void_p]
    for name, sig in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.restype = ctypes.c_int
        fn.argtypes = sig


# name -> argtypes for the simple (non-struct) entry points; filled by the modules that wrap them
_SIGNATURES: dict = {}


def register_signature(name: str, argtypes: list) -> None:
    _SIGNATURES[name] = argtypes
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.restype = ctypes.c_int
        fn.argtypes = argtypes


def available() -> bool:
    """True when CUDA is usable in this process (then the kernel library is required)."""
    return torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library; builds it first when it is missing and nvcc is present."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not LIB_PATH.exists() and os.environ.get("OLMAX_B200_NO_BUILD", "0") != "1":
            from ..csrc.build import build, find_nvcc

            if find_nvcc() is not None:
                build()
        if not LIB_PATH.exists():
            raise KernelError(
                f"kernel library {LIB_PATH} is missing: run `python -m olmax_b200.csrc.build` "
                "(the CUDA path never falls back to PyTorch math)"
            )
        handle = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _declare(handle)
        _LIB = handle
    return _LIB


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().ob_last_error()
        raise KernelError(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")


def stream_ptr(device: Optional[torch.device] = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_STATUS: dict = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] that kernels write when a bounded wait runs out (all zero = healthy)."""
    key = (device.type, device.index if (device.index is not None or device.type != "cuda") else torch.cuda.current_device())
    buf = _STATUS.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=device)
        _STATUS[key] = buf
    return buf


_STATUS_NAMES = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bad argument"}


def raise_for_status(vals) -> None:
    """Raise :class:`KernelError` when ``vals`` (the four status words: code, site, block, extra) report a failure."""
    if int(vals[0]) != 0:
        raise KernelError(f"kernel reported '{_STATUS_NAMES.get(int(vals[0]), int(vals[0]))}' at site {int(vals[1])}, "
                          f"block {int(vals[2])}, extra {int(vals[3])}")


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronising check of the kernel error words; raises KernelError when a kernel gave up on a wait."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    buf = status_buffer(device)
    vals = buf.tolist()
    if vals[0] != 0:
        buf.zero_()
        raise_for_status(vals)


def snapshot_status(device: torch.device):
    """Non-blocking copy of the status words, to be looked at later with :func:`resolve_status`: on a GPU the copy goes
    to pinned host memory behind everything already enqueued on the current stream, so reading it one step later costs
    no synchronisation.  (On a CPU device the buffer only exists for tests and is cloned.)"""
    buf = status_buffer(device)
    if not buf.is_cuda:
        return (buf.clone(), None)
    host = torch.empty(4, dtype=torch.int32, pin_memory=True)
    host.copy_(buf, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    return (host, ev)


def resolve_status(snapshot) -> None:
    """Wait for a :func:`snapshot_status` copy and raise :class:`KernelError` if it shows a failure."""
    host, ev = snapshot
    if ev is not None:
        ev.synchronize()
    raise_for_status(host.tolist())


class ObAttnArgs(ctypes.Structure):
    _fields_ = (
        [("q", ctypes.c_void_p), ("q_sb", ctypes.c_longlong), ("q_ss", ctypes.c_longlong), ("q_sh", ctypes.c_longlong)]
        + [("k", ctypes.c_void_p), ("k_sb", ctypes.c_longlong), ("k_ss", ctypes.c_longlong), ("k_sh", ctypes.c_longlong)]
        + [("v", ctypes.c_void_p), ("v_sb", ctypes.c_longlong), ("v_ss", ctypes.c_longlong), ("v_sh", ctypes.c_longlong)]
        + [("o", ctypes.c_void_p), ("o_sb", ctypes.c_longlong), ("o_ss", ctypes.c_longlong), ("o_sh", ctypes.c_longlong)]
        + [("lse", ctypes.c_void_p)]
        + [("d_o", ctypes.c_void_p), ("do_sb", ctypes.c_longlong), ("do_ss", ctypes.c_longlong), ("do_sh", ctypes.c_longlong)]
        + [("dq", ctypes.c_void_p), ("dq_sb", ctypes.c_longlong), ("dq_ss", ctypes.c_longlong), ("dq_sh", ctypes.c_longlong)]
        + [("dk", ctypes.c_void_p), ("dk_sb", ctypes.c_longlong), ("dk_ss", ctypes.c_longlong), ("dk_sh", ctypes.c_longlong)]
        + [("dv", ctypes.c_void_p), ("dv_sb", ctypes.c_longlong), ("dv_ss", ctypes.c_longlong), ("dv_sh", ctypes.c_longlong)]
        + [("delta", ctypes.c_void_p), ("dq_accum", ctypes.c_void_p)]
        + [("B", ctypes.c_int), ("S", ctypes.c_int), ("H", ctypes.c_int), ("Hkv", ctypes.c_int), ("D", ctypes.c_int)]
        + [("causal", ctypes.c_int), ("window", ctypes.c_int), ("scale", ctypes.c_float), ("softcap", ctypes.c_float)]
        + [("status", ctypes.c_void_p)]
        + [("Sk", ctypes.c_int), ("q_off", ctypes.c_int)]
    )

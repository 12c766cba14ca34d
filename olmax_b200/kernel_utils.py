"""
Availability checks for the native kernel library (the role ``olmax/te_utils.py:1-31`` plays for TransformerEngine in
the reference: an optional native dependency that features assert on before they use it).  Here the dependency is this
package's own ``lib/libolmax_b200.so``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

__all__ = ["kernels_available", "assert_kernels", "kernel_library_path", "host_library_path"]


def kernel_library_path() -> Path:
    from .csrc.build import LIB_PATH

    return LIB_PATH


def host_library_path() -> Path:
    from .csrc.build import CKPT_LIB_PATH

    return CKPT_LIB_PATH


def kernels_available() -> bool:
    """True when a CUDA device is visible and the sm_100a kernel library exists (or can be built: nvcc present)."""
    if not torch.cuda.is_available():
        return False
    if kernel_library_path().exists():
        return True
    from .csrc.build import find_nvcc

    return find_nvcc() is not None


def assert_kernels(feature: Optional[str] = None) -> None:
    """Raise a clear error when ``feature`` needs the CUDA kernels and they cannot be used on this machine."""
    if kernels_available():
        return
    what = f"{feature} requires" if feature else "This feature requires"
    if not torch.cuda.is_available():
        raise RuntimeError(f"{what} a CUDA device (sm_100a); none is visible.  The CPU path of every op is the PyTorch "
                           f"restatement in olmax_b200.ops.reference.")
    raise RuntimeError(f"{what} the kernel library {kernel_library_path()}, which is missing and cannot be built "
                       f"(nvcc not found).  Build it with `python -m olmax_b200.csrc.build`.")

"""
Initialisers (role of ``olmax/nn/init.py:10-63``).  Parameter initialisation itself happens inside
:meth:`ParamStore.init_parameters`, shard by shard from a per-parameter random stream, so that the values do not
depend on how the parameter is sharded; these functions are the stand-alone equivalents for user code and tests.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch


def truncated_normal(seed: int, shape: Sequence[int], stddev: float = 0.02, lower: float = -3.0, upper: float = 3.0,
                     dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None) -> torch.Tensor:
    """``stddev * TruncNormal(lower, upper)``: bounds are in units of ``stddev`` and the variate is not re-normalised."""
    gen = torch.Generator(device=device if device is not None else "cpu")
    gen.manual_seed(seed)
    t = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    torch.nn.init.trunc_normal_(t, 0.0, stddev, lower * stddev, upper * stddev, generator=gen)
    return t.to(dtype)


def zeros(shape: Sequence[int], dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
    return torch.zeros(tuple(shape), dtype=dtype, device=device)


def ones(shape: Sequence[int], dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
    return torch.ones(tuple(shape), dtype=dtype, device=device)

"""Debug helper: print a tensor's shape, dtype, device and how it is sharded (``olmax/debug.py:6-10``)."""

from __future__ import annotations

from typing import Any

import torch


def inspect(x: Any, name: str = "tensor") -> None:
    if isinstance(x, torch.Tensor):
        print(f"{name}: shape={tuple(x.shape)} dtype={x.dtype} device={x.device} stride={x.stride()}")
    elif hasattr(x, "describe"):
        print(f"{name}: {x.describe()}")
    else:
        print(f"{name}: {x!r}")

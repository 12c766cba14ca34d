"""
Functional API (``olmax/nn/functional.py``): weight-as-tensor versions of the ops for analysis and tests, evaluated
with the PyTorch restatement, plus the loss helpers.  Models call the handle-based ops in
:mod:`olmax_b200.ops.functional`, which dispatch to the CUDA kernels.
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from ..ops.reference import cross_entropy as cross_entropy_loss
from ..ops.reference import fused_cross_entropy as fused_cross_entropy_loss
from ..ops.reference import layer_norm, rms_norm

__all__ = ["linear", "layer_norm", "rms_norm", "cross_entropy_loss", "fused_cross_entropy_loss", "scan_module"]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ weight.t()
    return y + bias if bias is not None else y


def scan_module(layers: Sequence[Callable[[torch.Tensor], torch.Tensor]], x: torch.Tensor) -> torch.Tensor:
    """Apply a stack of identically-structured layers in sequence (``olmax/nn/functional.py:124-159``).  There is no
    trace/compile step here, so "scan" is a plain loop; its memory role (one layer's activations live at a time) is
    played by per-layer activation checkpointing."""
    for layer in layers:
        x = layer(x)
    return x

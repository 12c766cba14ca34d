"""Linear layer (``olmax/nn/linear.py:1-111``): weight ``(out, in)``, optional bias, FSDP on dim 0, optional TP split."""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import functional as F
from ..parallel import collectives as coll
from ..parallel.mesh import TPStyle
from .module import Module

__all__ = ["Linear"]


class Linear(Module):
    """
    ``y = x @ W^T (+ b)``.  ``tp_style``:

    * ``colwise``: output features split over the TP axis; the input is the full activation and the output carries
      ``out / tp`` features.
    * ``rowwise``: input features split over the TP axis; the output is a partial sum that the caller reduces
      (reduce-scatter under sequence parallelism, all-reduce otherwise).  A bias is not allowed under TP.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = False, tp_style: Optional[TPStyle] = None,
                 init_std: float = 0.02):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        tp = self.mesh.tp.size
        self.tp_style = TPStyle(tp_style) if (tp_style is not None and tp > 1) else None
        if self.tp_style is not None and bias:
            raise ValueError("bias is not supported together with tensor parallelism")
        tp_dim = None if self.tp_style is None else (0 if self.tp_style == TPStyle.colwise else 1)
        self.weight = self.add_param("weight", (out_features, in_features), tp_dim=tp_dim, init="trunc_normal",
                                     init_std=init_std)
        self.bias = self.add_param("bias", (out_features,), init="trunc_normal", init_std=init_std) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)

"""
Normalisation layers and their config (``olmax/nn/normalization.py:1-152``).  RMSNorm runs on the fused kernel with
optional residual fusion; LayerNorm has its own forward / backward kernels (residual adds stay ordinary tensor ops).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import functional as F
from ..ops import reference as ref
from ..utils.dataclass_codec import Registrable
from .module import Module

__all__ = ["Normalizer", "RMSNorm", "LayerNorm", "NormalizerConfig", "RMSNormConfig", "LayerNormConfig"]


class Normalizer(Module):
    def __init__(self, size: int, eps: float = 1e-5, use_weight: bool = True, use_bias: bool = False):
        super().__init__()
        self.size, self.eps = size, eps
        self.weight = self.add_param("weight", (size,), init="ones", decay=True) if use_weight else None
        self.bias = self.add_param("bias", (size,), init="zeros", decay=True) if use_bias else None


class RMSNorm(Normalizer):
    """``x * rsqrt(mean(x^2) + eps) * weight`` in fp32, cast back to the input dtype."""

    def __init__(self, size: int, eps: float = 1e-5, use_bias: bool = False):
        if use_bias:
            raise ValueError("RMSNorm with a bias is not supported")
        super().__init__(size, eps, use_weight=True, use_bias=False)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, mode: Optional[str] = None,
                heads: int = 1):
        """``mode`` None: norm(x); ``post``: residual + norm(x); ``pre``: returns (x + residual, norm(x + residual))."""
        return F.rms_norm(x, self.weight, self.eps, residual, mode, heads)


class LayerNorm(Normalizer):
    def __init__(self, size: int, eps: float = 1e-5, use_bias: bool = True):
        super().__init__(size, eps, use_weight=True, use_bias=use_bias)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, mode: Optional[str] = None,
                heads: int = 1):
        return F.layer_norm(x, self.weight, self.bias, self.eps, residual, mode, heads)


@dataclass
class NormalizerConfig(Registrable):
    eps: float = 1e-5
    use_bias: bool = False

    def build(self, size: int) -> Normalizer:
        raise NotImplementedError


@NormalizerConfig.register("rms_norm", default=True)
@dataclass
class RMSNormConfig(NormalizerConfig):
    def build(self, size: int) -> RMSNorm:
        return RMSNorm(size, eps=self.eps, use_bias=self.use_bias)


@NormalizerConfig.register("layer_norm")
@dataclass
class LayerNormConfig(NormalizerConfig):
    use_bias: bool = True

    def build(self, size: int) -> LayerNorm:
        return LayerNorm(size, eps=self.eps, use_bias=self.use_bias)

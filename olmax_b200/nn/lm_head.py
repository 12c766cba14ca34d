"""
LM head (``olmax/nn/lm_head.py:1-61``).  ``forward`` returns fp32 logits like the reference; training uses
:meth:`LMHead.loss`, which fuses the projection with the cross entropy so that the ``[tokens, vocab]`` logits are
only ever materialised a chunk of rows at a time.  ``tied_weight`` lets the head share the embedding matrix.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..ops import functional as F
from ..ops import reference as ref
from .linear import Linear
from .module import Module, current_build_context

__all__ = ["LMHead", "LMHeadConfig"]


class LMHead(Module):
    def __init__(self, d_model: int, vocab_size: int, bias: bool = False, tied_weight=None,
                 logit_softcap: Optional[float] = None, init_std: float = 0.02):
        super().__init__()
        if bias:
            raise ValueError("LMHead bias is not supported by the fused loss")
        self.vocab_size = vocab_size
        self.logit_softcap = logit_softcap
        self.proj: Optional[Linear] = None
        if tied_weight is None:
            with current_build_context().scope("proj"):
                self.proj = Linear(d_model, vocab_size, init_std=init_std)
            self._weight = self.proj.weight
        else:
            self._weight = tied_weight

    @property
    def weight(self):
        return self._weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = F.linear(x, self._weight).float()
        return ref.softcap(logits, self.logit_softcap or 0.0)

    def loss(self, x: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, z_loss_multiplier: float = 0.0,
             chunk_rows: int = 2048) -> Tuple[torch.Tensor, torch.Tensor]:
        return F.linear_cross_entropy(x, self._weight, labels, ignore_index, self.logit_softcap or 0.0,
                                      z_loss_multiplier, chunk_rows)


@dataclass
class LMHeadConfig:
    bias: bool = False
    logit_softcap: Optional[float] = None

    def build(self, d_model: int, vocab_size: int, tied_weight=None, init_std: float = 0.02) -> LMHead:
        return LMHead(d_model, vocab_size, self.bias, tied_weight, self.logit_softcap, init_std)

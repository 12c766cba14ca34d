"""
LM head (``olmax/nn/lm_head.py:1-61``).  ``forward`` returns fp32 logits like the reference; training uses
:meth:`LMHead.loss`, which fuses the projection with the cross entropy so that the ``[tokens, vocab]`` logits are
only ever materialised a chunk of rows at a time.  ``tied_weight`` lets the head share the embedding matrix.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..exceptions import OLMaxConfigurationError
from ..ops import functional as F
from ..ops import reference as ref
from ..parallel import collectives as coll
from ..parallel.mesh import TPStyle
from .linear import Linear
from .module import Module, current_build_context

__all__ = ["LMHead", "LMHeadConfig"]


class LMHead(Module):
    def __init__(self, d_model: int, vocab_size: int, bias: bool = False, tied_weight=None,
                 logit_softcap: Optional[float] = None, init_std: float = 0.02, vocab_parallel: bool = False):
        super().__init__()
        if bias:
            raise ValueError("LMHead bias is not supported by the fused loss")
        self.vocab_size = vocab_size
        self.logit_softcap = logit_softcap
        self.proj: Optional[Linear] = None
        # vocabulary parallelism: the head's rows (classes) are split over the tensor-parallel group
        self.vocab_parallel = bool(vocab_parallel) and self.mesh.tp.size > 1
        if self.vocab_parallel and tied_weight is not None:
            raise OLMaxConfigurationError("a vocabulary-parallel LM head cannot share the (unsplit) embedding matrix")
        if tied_weight is None:
            with current_build_context().scope("proj"):
                self.proj = Linear(d_model, vocab_size, init_std=init_std,
                                   tp_style=TPStyle.colwise if self.vocab_parallel else None)
            self._weight = self.proj.weight
        else:
            self._weight = tied_weight

    @property
    def weight(self):
        return self._weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.vocab_parallel:
            # every member computes its vocabulary slice for the gathered rows; the slices are concatenated and each
            # member keeps the logits of its own rows
            tp = self.mesh.tp
            rows = x.shape[0]
            part = F.linear(coll.all_gather(x.contiguous(), tp, dim=0), self._weight).float()
            logits = coll.all_gather(part.contiguous(), tp, dim=1)[tp.rank * rows : (tp.rank + 1) * rows]
        else:
            logits = F.linear(x, self._weight).float()
        return ref.softcap(logits, self.logit_softcap or 0.0)

    def loss(self, x: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, z_loss_multiplier: float = 0.0,
             chunk_rows: int = 2048) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.vocab_parallel:
            tpc = self.store.tp_symm if x.is_cuda else None
            return F.vocab_parallel_linear_cross_entropy(x, self._weight, labels, self.mesh.tp, tpc, ignore_index,
                                                         self.logit_softcap or 0.0, z_loss_multiplier, chunk_rows)
        return F.linear_cross_entropy(x, self._weight, labels, ignore_index, self.logit_softcap or 0.0,
                                      z_loss_multiplier, chunk_rows)


@dataclass
class LMHeadConfig:
    bias: bool = False
    logit_softcap: Optional[float] = None
    vocab_parallel: bool = False
    """Split the head's vocabulary over the tensor-parallel axis and compute the loss from the members' slices
    (``ops/functional.py: vocab_parallel_linear_cross_entropy``); no effect on a mesh without a TP axis."""

    def build(self, d_model: int, vocab_size: int, tied_weight=None, init_std: float = 0.02) -> LMHead:
        return LMHead(d_model, vocab_size, self.bias, tied_weight, self.logit_softcap, init_std, self.vocab_parallel)

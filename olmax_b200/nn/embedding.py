"""Token embedding (``olmax/nn/embedding.py:1-32``): weight ``(vocab, d)`` sharded over the vocabulary."""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import functional as F
from .module import Module

__all__ = ["Embedding"]


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, scale: float = 1.0, init_std: float = 0.02):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.scale = num_embeddings, embedding_dim, scale
        self.weight = self.add_param("weight", (num_embeddings, embedding_dim), init="trunc_normal", init_std=init_std)

    def forward(self, ids: torch.Tensor, anchor: Optional[torch.Tensor] = None) -> torch.Tensor:
        return F.embedding(ids, self.weight, self.scale, anchor)

"""Rotary position embedding (``olmax/nn/rope.py:1-145``), rotate-half convention, tables precomputed in fp32."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..ops import functional as F
from ..ops import reference as ref

__all__ = ["RotaryPositionalEmbedding", "RotaryPositionalEmbeddingConfig", "BufferCache"]


class BufferCache(dict):
    """Precomputed (cos, sin) tables keyed by ``(head_dim, seq_len, theta)`` (``olmax/nn/rope.py:91-97``)."""


class RotaryPositionalEmbedding(torch.nn.Module):
    def __init__(self, head_dim: int, theta: float = 10000.0):
        super().__init__()
        self.head_dim, self.theta = head_dim, float(theta)

    def get_tables(self, seq_len: int, device, cache: Optional[BufferCache] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        key = (self.head_dim, seq_len, self.theta, str(device))
        if cache is not None and key in cache:
            return cache[key]
        cos, sin = ref.rope_tables(seq_len, self.head_dim, self.theta, device=device)
        if cache is not None:
            cache[key] = (cos, sin)
        return cos, sin

    def get_local_tables(self, local_len: int, cp_size: int, cp_rank: int, device,
                         cache: Optional[BufferCache] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Rows of the full-sequence tables at the positions a context-parallel rank holds
        (``olmax/nn/rope.py:135-143``)."""
        from ..parallel.context import cp_local_positions

        key = (self.head_dim, local_len, self.theta, str(device), cp_size, cp_rank)
        if cache is not None and key in cache:
            return cache[key]
        cos, sin = self.get_tables(local_len * cp_size, device, cache)
        pos = cp_local_positions(local_len * cp_size, cp_size, cp_rank, device=cos.device)
        out = (cos.index_select(0, pos).contiguous(), sin.index_select(0, pos).contiguous())
        if cache is not None:
            cache[key] = out
        return out

    def tables_for(self, local_len: int, device, cache: Optional[BufferCache] = None, cp_size: int = 1,
                   cp_rank: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        """The (cos, sin) rows for this rank's ``local_len`` tokens (all of the sequence without context parallelism)."""
        if cp_size > 1:
            return self.get_local_tables(local_len, cp_size, cp_rank, device, cache)
        return self.get_tables(local_len, device, cache)

    def forward(self, x: torch.Tensor, cache: Optional[BufferCache] = None, cp_size: int = 1, cp_rank: int = 0) -> torch.Tensor:
        """x: [B, S, H, D] (S = this rank's tokens under context parallelism)."""
        cos, sin = self.tables_for(x.shape[1], x.device, cache, cp_size, cp_rank)
        return F.rope(x, cos, sin)


@dataclass
class RotaryPositionalEmbeddingConfig:
    theta: float = 10000.0

    def build(self, head_dim: int) -> RotaryPositionalEmbedding:
        return RotaryPositionalEmbedding(head_dim, self.theta)

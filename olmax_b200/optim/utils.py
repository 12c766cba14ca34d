"""Gradient clipping helpers and state extraction (``olmax/optim/utils.py:11-60``)."""

from __future__ import annotations

from typing import Any, Tuple

import torch

from ..utils.tree import get_global_norm, tree_map

__all__ = ["clip_grads_by_global_norm", "extract_state", "extract_hyperparameter"]


def clip_grads_by_global_norm(grads: Any, max_norm: float) -> Tuple[Any, torch.Tensor]:
    """``g * max_norm / max(max_norm, |g|)`` over a tree of tensors; also returns the norm."""
    norm = get_global_norm(grads)
    coef = max_norm / torch.clamp(norm, min=max_norm)
    return tree_map(lambda g: g * coef.to(g.dtype), grads), norm


def extract_state(optim, name: str):
    """Look a named entry up in an optimizer's state (``count``, ``exp_avg``, ...)."""
    state = optim.state_dict()
    if name not in state:
        raise KeyError(f"optimizer state has no entry '{name}'; entries: {sorted(state)}")
    return state[name]


def extract_hyperparameter(optim, name: str) -> float:
    return optim.hyperparameters()[name]

"""Numeric comparison helper for tests (``olmax/testing/utils.py:13-15``)."""

import torch


def allclose(a: torch.Tensor, b: torch.Tensor, rtol: float = 1e-3, atol: float = 1e-5) -> bool:
    return bool(torch.allclose(a.float().cpu(), b.float().cpu(), rtol=rtol, atol=atol))


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-30))

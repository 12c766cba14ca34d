"""
Collective wrappers over a mesh-axis group (role of the explicit collectives in
``olmax/distributed/parallel.py:409-436``): tiled all-gather, reduce-scatter and all-reduce with the reference's
pre-divide rule for low-precision sums, plus the two sequence-parallel autograd pairs used by tensor parallelism
(all-gather whose backward is a reduce-scatter, and the reverse).

Every function is a no-op on a group of one, uses NCCL on CUDA tensors, and falls back to gloo-compatible
formulations on CPU (gloo has no reduce-scatter: all-reduce then slice).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .dist_utils import get_reduce_divide_factor

__all__ = [
    "all_gather",
    "all_gather_into",
    "reduce_scatter",
    "reduce_scatter_into",
    "all_reduce",
    "SeqAllGather",
    "SeqReduceScatter",
    "seq_all_gather",
    "seq_reduce_scatter",
    "copy_to_tp_region",
]


def _region(label: str):
    """Device-time bracket of a collective when kernel timing is on (``ops.kernels.timed_region``)."""
    from ..ops import kernels as K

    return K.timed_region(label)


def _is_gloo(group) -> bool:
    try:
        return dist.get_backend(group.pg) == "gloo"
    except Exception:
        return False


def all_gather_into(out: torch.Tensor, x: torch.Tensor, group, async_op: bool = False):
    """``out`` (group.size * x.numel(), rank-major) <- concatenation of every rank's ``x``."""
    if group.size == 1:
        out.view(-1).copy_(x.reshape(-1))
        return None
    if _is_gloo(group):
        chunks = list(out.view(group.size, -1).unbind(0))
        return dist.all_gather(chunks, x.reshape(-1).contiguous(), group=group.pg, async_op=async_op)
    return dist.all_gather_into_tensor(out.view(-1), x.reshape(-1).contiguous(), group=group.pg, async_op=async_op)


def all_gather(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
    """Tiled all-gather along ``dim``."""
    if group.size == 1:
        return x
    xm = x.movedim(dim, 0).contiguous()
    out = torch.empty((group.size * xm.shape[0],) + tuple(xm.shape[1:]), dtype=x.dtype, device=x.device)
    all_gather_into(out, xm, group)
    return out.movedim(0, dim) if dim != 0 else out


def reduce_scatter_into(out: torch.Tensor, x: torch.Tensor, group, mean: bool = False, predivide: bool = True):
    """
    ``out`` <- this rank's slice of the sum (or mean) of ``x`` over the group; ``x`` is rank-major
    (group.size * out.numel()).  With ``predivide`` and a 16-bit dtype the summands are divided by
    ``get_reduce_divide_factor(n)`` first and the result rescaled, which keeps partial sums in range.
    """
    n = group.size
    if n == 1:
        out.view(-1).copy_(x.reshape(-1))
        return out
    low_precision = x.dtype in (torch.bfloat16, torch.float16)
    f = get_reduce_divide_factor(n) if (predivide and low_precision) else 1
    xin = x.reshape(-1)
    if f != 1:
        xin = xin / f
    if _is_gloo(group):
        buf = xin.clone() if xin.data_ptr() == x.data_ptr() else xin
        dist.all_reduce(buf, group=group.pg)
        out.view(-1).copy_(buf.view(n, -1)[group.rank])
    else:
        dist.reduce_scatter_tensor(out.view(-1), xin.contiguous(), group=group.pg)
    post = f / n if mean else float(f)
    if post != 1.0:
        out.mul_(post)
    return out


def reduce_scatter(x: torch.Tensor, group, dim: int = 0, mean: bool = False) -> torch.Tensor:
    if group.size == 1:
        return x
    xm = x.movedim(dim, 0).contiguous()
    assert xm.shape[0] % group.size == 0, "reduce_scatter: dimension not divisible by the group size"
    out = torch.empty((xm.shape[0] // group.size,) + tuple(xm.shape[1:]), dtype=x.dtype, device=x.device)
    reduce_scatter_into(out, xm, group, mean=mean)
    return out.movedim(0, dim) if dim != 0 else out


def all_reduce(x: torch.Tensor, group, mean: bool = False, predivide: bool = True) -> torch.Tensor:
    """In-place sum (or mean) over the group."""
    n = group.size
    if n == 1:
        return x
    low_precision = x.dtype in (torch.bfloat16, torch.float16)
    f = get_reduce_divide_factor(n) if (predivide and low_precision) else 1
    if f != 1:
        x.div_(f)
    dist.all_reduce(x, group=group.pg)
    post = f / n if mean else float(f)
    if post != 1.0:
        x.mul_(post)
    return x


class SeqAllGather(torch.autograd.Function):
    """[M/n, d] -> [M, d] over the group; backward reduce-scatters (sequence-parallel entry of a TP region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        with _region("nccl seq all_gather"):
            return all_gather(x, group, dim=0)

    @staticmethod
    def backward(ctx, dy):
        with _region("nccl seq reduce_scatter"):
            return reduce_scatter(dy.contiguous(), ctx.group, dim=0), None


class SeqReduceScatter(torch.autograd.Function):
    """[M, d] partial sums -> [M/n, d] over the group; backward all-gathers (sequence-parallel exit of a TP region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        with _region("nccl seq reduce_scatter"):
            return reduce_scatter(x.contiguous(), group, dim=0)

    @staticmethod
    def backward(ctx, dy):
        with _region("nccl seq all_gather"):
            return all_gather(dy.contiguous(), ctx.group, dim=0), None


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (TP without sequence parallelism)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        return all_reduce(dy.contiguous(), ctx.group), None


def seq_all_gather(x: torch.Tensor, group) -> torch.Tensor:
    return x if group.size == 1 else SeqAllGather.apply(x, group)


def seq_reduce_scatter(x: torch.Tensor, group) -> torch.Tensor:
    return x if group.size == 1 else SeqReduceScatter.apply(x, group)


def copy_to_tp_region(x: torch.Tensor, group) -> torch.Tensor:
    return x if group.size == 1 else _CopyToTP.apply(x, group)

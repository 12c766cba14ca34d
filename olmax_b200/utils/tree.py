"""
Helpers over nested containers of tensors ("trees": dicts / lists / tuples of ``torch.Tensor``), the PyTorch
counterparts of ``olmax/jax_utils.py:15-135``: casting, zeros-like, parameter counting, global norm, peak device
memory, deterministic per-shape RNG streams.
"""

from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

__all__ = [
    "tree_map",
    "tree_leaves",
    "tree_flatten_with_paths",
    "cast_tree",
    "zeros_like_tree",
    "count_params",
    "get_global_norm",
    "get_peak_local_device_memory_usage",
    "get_cudnn_version",
    "fold_in",
    "split_seed",
    "shaped_rng_split",
    "maybe_rng_split",
    "vmap_multiple",
    "abs_sq",
    "is_in_jit",
    "uncommit_single_device_arrays",
    "with_optional_sharding_contraint",
]


def tree_map(fn: Callable[[torch.Tensor], Any], tree: Any) -> Any:
    if isinstance(tree, torch.Tensor):
        return fn(tree)
    if isinstance(tree, dict):
        return {k: tree_map(fn, v) for k, v in tree.items()}
    if isinstance(tree, tuple):
        return tuple(tree_map(fn, v) for v in tree)
    if isinstance(tree, list):
        return [tree_map(fn, v) for v in tree]
    return tree


def tree_leaves(tree: Any) -> List[torch.Tensor]:
    return [t for _, t in tree_flatten_with_paths(tree)]


def tree_flatten_with_paths(tree: Any, prefix: str = "") -> List[Tuple[str, torch.Tensor]]:
    out: List[Tuple[str, torch.Tensor]] = []
    if isinstance(tree, torch.Tensor):
        out.append((prefix, tree))
    elif isinstance(tree, dict):
        for k in tree:
            out.extend(tree_flatten_with_paths(tree[k], f"{prefix}.{k}" if prefix else str(k)))
    elif isinstance(tree, (list, tuple)):
        for i, v in enumerate(tree):
            out.extend(tree_flatten_with_paths(v, f"{prefix}.{i}" if prefix else str(i)))
    return out


def cast_tree(tree: Any, dtype: torch.dtype) -> Any:
    """Cast every floating-point leaf to ``dtype`` (integer leaves are left alone)."""
    return tree_map(lambda t: t.to(dtype) if t.is_floating_point() else t, tree)


def zeros_like_tree(tree: Any) -> Any:
    return tree_map(torch.zeros_like, tree)


def count_params(tree: Any) -> Tuple[int, int]:
    """(number of elements, bytes) over all leaves."""
    n = b = 0
    for t in tree_leaves(tree):
        n += t.numel()
        b += t.numel() * t.element_size()
    return n, b


def get_global_norm(tree: Any) -> torch.Tensor:
    """sqrt of the sum of squared entries over every leaf (computed in fp32)."""
    leaves = tree_leaves(tree)
    if not leaves:
        return torch.zeros(())
    total = torch.zeros((), dtype=torch.float32, device=leaves[0].device)
    for t in leaves:
        total = total + t.float().pow(2).sum()
    return total.sqrt()


def get_peak_local_device_memory_usage(device: Optional[torch.device] = None) -> Optional[int]:
    """Peak bytes allocated on the local CUDA device, or None on CPU."""
    if not torch.cuda.is_available():
        return None
    return int(torch.cuda.max_memory_allocated(device))


def get_cudnn_version() -> Optional[int]:
    try:
        return torch.backends.cudnn.version()
    except Exception:
        return None


_MASK64 = (1 << 64) - 1


def fold_in(seed: int, data: int) -> int:
    """Derive a new 63-bit seed from ``seed`` and an integer (splitmix64 mixing); deterministic across ranks."""
    z = (seed + 0x9E3779B97F4A7C15 * (data + 1)) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z = z ^ (z >> 31)
    return z & ((1 << 63) - 1)


def split_seed(seed: int, n: int) -> List[int]:
    return [fold_in(seed, i) for i in range(n)]


def shaped_rng_split(seed: int, shape: Sequence[int]) -> Any:
    """Nested lists of seeds with the given shape (``olmax/jax_utils.py`` ``shaped_rng_split``)."""
    if len(shape) == 0:
        return seed
    return [shaped_rng_split(fold_in(seed, i), shape[1:]) for i in range(shape[0])]


def maybe_rng_split(seed: Optional[int], num: int = 2) -> List[Optional[int]]:
    """``num`` seeds derived from ``seed``, or ``num`` Nones when there is no seed (``olmax/jax_utils.py:127-135``)."""
    if seed is None:
        return [None] * num
    return split_seed(seed, num)


def vmap_multiple(fun: Callable, n: int) -> Callable:
    """``fun`` vectorised over ``n`` leading dimensions (``olmax/jax_utils.py:15-21``; ``torch.func.vmap`` applied n times)."""
    for _ in range(n):
        fun = torch.func.vmap(fun)
    return fun


def abs_sq(x: torch.Tensor) -> torch.Tensor:
    """|x|^2 without a square root, also for complex tensors (``olmax/jax_utils.py:93-102``)."""
    if x.is_complex():
        return x.real.square() + x.imag.square()
    return x.square()


def is_in_jit() -> bool:
    """True while a graph compiler traces the caller (``olmax/jax_utils.py:76-77``).  The hot path here is eager kernels
    on streams, so this is only ever true when a user wraps something in ``torch.compile`` themselves."""
    try:
        return bool(torch.compiler.is_compiling())
    except Exception:
        return False


def uncommit_single_device_arrays(tree: Any) -> Any:
    """Accepted for source compatibility (``olmax/jax_utils.py:32-44``): JAX arrays can be "committed" to a device, which
    restricts where later computations may run; PyTorch tensors have no such state, so the tree is returned as is."""
    return tree


def with_optional_sharding_contraint(tree: Any, sharding: Any = None, cond: Optional[Callable[[torch.Tensor], bool]] = None) -> Any:
    """Accepted for source compatibility (``olmax/jax_utils.py:61-73``, spelling as in the reference): a sharding
    constraint is a hint to an SPMD partitioner.  Here every process holds exactly its shard and placement is explicit
    (``parallel/param_store.py``), so there is nothing to constrain and the tree is returned as is."""
    return tree

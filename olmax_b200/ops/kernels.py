"""
Thin Python wrappers around the C entry points of the sm_100a kernel library.  They take CUDA tensors, check the
layout rules the kernels rely on (bf16, 16-byte alignment, strides that are multiples of 8 elements), build the
argument structs and launch on the current stream.  No math happens here and there is no PyTorch fallback: on a
machine with a GPU a missing library raises.

A launch counter (:func:`launch_count`) records how many of our kernels were enqueued, which the benchmark reports.
"""

from __future__ import annotations

import contextlib
import ctypes
import functools
import math
import os
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import KernelError, ObAttnArgs, ObGemmArgs, check, lib, register_signature, status_buffer, stream_ptr

__all__ = [
    "EPI_BF16", "EPI_F32", "EPI_F32_ACC", "EPI_F32_RED", "EPI_SWIGLU", "EPI_GEGLU", "EPI_BF16_ACC",
    "gemm", "flash_attn_fwd", "flash_attn_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "rmsnorm_rope_fwd", "rmsnorm_rope_bwd", "rope", "glu_fwd", "glu_bwd",
    "embed_gather", "embed_scatter", "ce_fwd_bwd", "ce_vp_stats", "ce_vp_grad", "count_valid", "adamw", "sumsq", "clip_coef", "cast_f32_bf16",
    "layernorm_fwd", "layernorm_bwd", "gather_shards", "scatter_add_shards", "allreduce_p2p", "allreduce_multimem",
    "peer_barrier", "peer_signal", "peer_wait", "copy_bytes", "push_copy", "fold_slots_bf16", "reduce_slots",
    "launch_count", "reset_launch_count", "pointer_table",
    "timing_enabled", "set_timing", "timed_region", "timing_report", "format_timing",
]

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_F32_RED, EPI_SWIGLU, EPI_GEGLU, EPI_BF16_ACC = range(7)

_LAUNCHES = 0


def launch_count() -> int:
    return _LAUNCHES


def reset_launch_count() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


_vp = ctypes.c_void_p
_ll = ctypes.c_longlong
_i = ctypes.c_int
_f = ctypes.c_float

register_signature("ob_rmsnorm_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _ll, _ll, _ll, _i, _f, _vp])
register_signature("ob_rmsnorm_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _ll, _ll, _ll, _f, _vp])
register_signature("ob_layernorm_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _f, _vp])
register_signature("ob_layernorm_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _f, _vp])
register_signature("ob_rope", [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll, _f, _i, _vp])
register_signature("ob_rmsnorm_rope_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _ll, _ll, _i, _f, _vp])
register_signature("ob_rmsnorm_rope_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _ll, _ll, _ll, _i, _f, _vp])
register_signature("ob_glu_fwd", [_vp, _vp, _vp, _ll, _i, _vp])
register_signature("ob_glu_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _vp])
register_signature("ob_embed_gather", [_vp, _vp, _i, _i, _vp, _ll, _i, _f, _vp])
register_signature("ob_embed_scatter", [_vp, _vp, _i, _i, _vp, _ll, _i, _f, _vp])
register_signature("ob_ce_fwd_bwd", [_vp, _ll, _vp, _vp, _ll, _vp, _vp, _vp, _ll, _i, _i, _f, _f, _f, _vp])
register_signature("ob_ce_vp_stats", [_vp, _ll, _vp, _vp, _ll, _i, _ll, _f, _vp])
register_signature("ob_ce_vp_grad", [_vp, _ll, _vp, _vp, _ll, _vp, _i, _vp, _ll, _ll, _i, _vp, _ll, _i, _ll, _ll, _i, _f, _f, _f, _vp])
register_signature("ob_count_valid", [_vp, _ll, _i, _i, _vp, _vp, _vp])
register_signature("ob_adamw", [_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _vp, _i, _vp])
register_signature("ob_sumsq", [_vp, _ll, _vp, _vp])
register_signature("ob_clip_coef", [_vp, _f, _f, _vp, _vp])
register_signature("ob_cast_f32_bf16", [_vp, _vp, _ll, _vp])
register_signature("ob_peer_barrier", [_vp, _i, _i, ctypes.c_uint, _ll, _vp, _vp])
register_signature("ob_peer_signal", [_vp, _i, _i, ctypes.c_uint, _vp])
register_signature("ob_peer_wait", [_vp, _i, _i, ctypes.c_uint, _ll, _vp, _vp])
register_signature("ob_copy_bytes", [_vp, _vp, _ll, _i, _i, _vp])
register_signature("ob_push_copy", [_vp, _vp, _ll, _i, _i, _i, _vp])
register_signature("ob_fold_slots_bf16", [_vp, _vp, _ll, _i, _ll, _i, _i, _vp])
register_signature("ob_gather_shards", [_vp, _vp, _ll, _ll, _i, _i, _vp])
register_signature("ob_scatter_add_shards", [_vp, _vp, _ll, _i, _f, _vp])
register_signature("ob_allreduce_p2p_f32", [_vp, _ll, _i, _i, _f, _i, _vp])
register_signature("ob_allreduce_multimem_f32", [_vp, _ll, _i, _i, _i, _vp])
register_signature("ob_reduce_slots_f32", [_vp, _vp, _ll, _i, _ll, _f, _vp])
register_signature("ob_reduce_slots_bf16", [_vp, _vp, _ll, _i, _ll, _f, _vp])


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _req_bf16(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_cuda):
            raise KernelError(f"expected a CUDA bf16 tensor, got {t.dtype} on {t.device}")


def pointer_table(ptrs: Sequence[int], device: torch.device) -> torch.Tensor:
    """int64 CUDA tensor holding raw pointers (what the kernels take as ``T* const*``)."""
    return torch.tensor(list(ptrs), dtype=torch.int64, device=device)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    M: int,
    N: int,
    K: int,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    epi: int = EPI_BF16,
    alpha: float = 1.0,
    lda: Optional[int] = None,
    ldb: Optional[int] = None,
    ldc: Optional[int] = None,
    b_shard_stride: int = 0,
    N_s: int = 0,
    Kc_s: int = 0,
    M_s: int = 0,
    b2: Optional[torch.Tensor] = None,
    c2: Optional[torch.Tensor] = None,
    c3: Optional[torch.Tensor] = None,
    c_shards: Optional[torch.Tensor] = None,
    c_shard_stride: int = 0,
    max_ctas: int = 0,
    ag_src: Optional[torch.Tensor] = None,
    ag_src2: Optional[torch.Tensor] = None,
    ag_flags: Optional[torch.Tensor] = None,
    ag_rank: int = 0,
    prefetch: Optional[tuple] = None,
    no_tma_epilogue: bool = False,
    group_m: int = 0,
    multi_box_mn: bool = False,
    m_shard_rot: int = 0,
    ag_on_a: bool = False,
    no_split_k: bool = False,
) -> None:
    """``C[M, N] (+)= alpha * A[M, K] . B[K, N]``; see ``csrc/gemm.h`` for operand layouts and sharding."""
    _req_bf16(a, b, b2)
    args = ObGemmArgs()
    args.a = a.data_ptr()
    args.lda = lda if lda is not None else a.stride(0)
    args.b = b.data_ptr()
    args.ldb = ldb if ldb is not None else b.stride(0)
    args.b_shard_stride = b_shard_stride
    args.b2 = _ptr(b2)
    args.c = c.data_ptr()
    args.ldc = ldc if ldc is not None else c.stride(0)
    args.c2 = _ptr(c2)
    args.c3 = _ptr(c3)
    args.c_shards = _ptr(c_shards)
    args.c_shard_stride = c_shard_stride
    args.M, args.N, args.Kc = M, N, K
    args.M_s, args.N_s, args.Kc_s = M_s, N_s, Kc_s
    args.a_mn, args.b_mn, args.epi, args.alpha = int(a_mn), int(b_mn), epi, alpha
    args.status = status_buffer(a.device).data_ptr()
    args.max_ctas = max_ctas
    args.ag_src = _ptr(ag_src)
    args.ag_src2 = _ptr(ag_src2)
    args.ag_flags = _ptr(ag_flags)
    args.ag_rank = ag_rank
    args.no_tma_epilogue = int(no_tma_epilogue)
    args.group_m = group_m
    args.m_shard_rot = m_shard_rot
    args.multi_box_mn = int(multi_box_mn)
    args.ag_on_a = int(ag_on_a)
    args.no_split_k = int(no_split_k)
    if prefetch is not None:
        table, dst_ptr, dst_stride, off, nbytes, shards, rank = prefetch
        args.pf_src, args.pf_dst, args.pf_dst_stride = table.data_ptr(), dst_ptr, dst_stride
        args.pf_off, args.pf_bytes, args.pf_shards, args.pf_rank = off, nbytes, shards, rank
    check(lib().ob_gemm_bf16(ctypes.byref(args), stream_ptr(a.device)), "gemm")
    _count()


def _set_bshd(args: ObAttnArgs, field: str, t: torch.Tensor, prefix: Optional[str] = None) -> None:
    prefix = prefix or field
    if t.stride(-1) != 1:
        raise KernelError("attention tensors need a contiguous head dimension")
    setattr(args, field, t.data_ptr())
    setattr(args, prefix + "_sb", t.stride(0))
    setattr(args, prefix + "_ss", t.stride(1))
    setattr(args, prefix + "_sh", t.stride(2))


def flash_attn_fwd(q, k, v, *, causal=True, window=-1, softcap=0.0, scale=None, q_off=0) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,S,H,128], k/v [B,Sk,Hkv,128] -> (o [B,S,H,128] bf16, lse [B,H,S] fp32).  Query row i sits at position
    ``q_off + i`` of the key axis (rectangular problems of context-parallel / blockwise attention)."""
    _req_bf16(q, k, v)
    B, S, H, D = q.shape
    o = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    a = ObAttnArgs()
    _set_bshd(a, "q", q)
    _set_bshd(a, "k", k)
    _set_bshd(a, "v", v)
    _set_bshd(a, "o", o)
    a.lse = lse.data_ptr()
    a.B, a.S, a.H, a.Hkv, a.D = B, S, H, k.shape[2], D
    a.causal, a.window = int(causal), int(window)
    a.Sk, a.q_off = k.shape[1], int(q_off)
    a.scale = scale if scale is not None else 1.0 / math.sqrt(D)
    a.softcap = float(softcap)
    a.status = status_buffer(q.device).data_ptr()
    check(lib().ob_flash_attn_fwd(ctypes.byref(a), stream_ptr(q.device)), "flash_attn_fwd")
    _count()
    return o, lse


def flash_attn_bwd(q, k, v, o, lse, d_o, *, causal=True, window=-1, softcap=0.0, scale=None,
                   dq=None, dk=None, dv=None, q_off=0):
    _req_bf16(q, k, v, o, d_o)
    B, S, H, D = q.shape
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    acc = torch.empty((B, S, H, D), dtype=torch.float32, device=q.device)
    a = ObAttnArgs()
    _set_bshd(a, "q", q)
    _set_bshd(a, "k", k)
    _set_bshd(a, "v", v)
    _set_bshd(a, "o", o)
    _set_bshd(a, "d_o", d_o, "do")
    _set_bshd(a, "dq", dq)
    _set_bshd(a, "dk", dk)
    _set_bshd(a, "dv", dv)
    a.lse = lse.data_ptr()
    a.delta = delta.data_ptr()
    a.dq_accum = acc.data_ptr()
    a.B, a.S, a.H, a.Hkv, a.D = B, S, H, k.shape[2], D
    a.causal, a.window = int(causal), int(window)
    a.Sk, a.q_off = k.shape[1], int(q_off)
    a.scale = scale if scale is not None else 1.0 / math.sqrt(D)
    a.softcap = float(softcap)
    a.status = status_buffer(q.device).data_ptr()
    check(lib().ob_flash_attn_bwd(ctypes.byref(a), stream_ptr(q.device)), "flash_attn_bwd")
    _count(3)
    return dq, dk, dv


def rmsnorm_fwd(x, w, y, *, rows, d, eps, res=None, sum_out=None, rstd=None, heads=1, ld_x=None, ld_res=None,
                ld_y=None, add_before=False) -> None:
    _req_bf16(x, w, y, res, sum_out)
    check(lib().ob_rmsnorm_fwd(x.data_ptr(), _ptr(res), w.data_ptr(), y.data_ptr(), _ptr(sum_out), _ptr(rstd), rows, d,
                               heads, ld_x if ld_x is not None else d, ld_res if ld_res is not None else d,
                               ld_y if ld_y is not None else d, int(add_before), eps, stream_ptr(x.device)), "rmsnorm_fwd")
    _count()


def rmsnorm_bwd(dy, x, w, rstd, dx, *, rows, d, dw=None, dsum=None, heads=1, ld_dy=None, ld_x=None, ld_dx=None,
                dw_scale=1.0) -> None:
    _req_bf16(dy, x, w, dx, dsum)
    check(lib().ob_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ptr(dsum), dx.data_ptr(),
                               _ptr(dw), rows, d, heads, ld_dy if ld_dy is not None else d,
                               ld_x if ld_x is not None else d, ld_dx if ld_dx is not None else d, dw_scale,
                               stream_ptr(x.device)), "rmsnorm_bwd")
    _count()


def rmsnorm_rope_fwd(x, w, y, rstd, cos, sin, *, rows, d, hd, heads, seq_len, eps, ld_x=None, ld_y=None) -> None:
    """y = rope(rmsnorm(x) * w): rows of ``d`` elements (``d / hd`` heads each), table row ``(row / heads) % seq_len``."""
    _req_bf16(x, w, y)
    check(lib().ob_rmsnorm_rope_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), _ptr(rstd), cos.data_ptr(), sin.data_ptr(),
                                    rows, d, hd, heads, ld_x if ld_x is not None else d, ld_y if ld_y is not None else d,
                                    seq_len, eps, stream_ptr(x.device)), "rmsnorm_rope_fwd")
    _count()


def rmsnorm_rope_bwd(dy, x, w, rstd, dx, cos, sin, *, rows, d, hd, heads, seq_len, dw=None, dw_scale=1.0, ld_dy=None,
                     ld_x=None, ld_dx=None) -> None:
    _req_bf16(dy, x, w, dx)
    check(lib().ob_rmsnorm_rope_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), _ptr(dw),
                                    cos.data_ptr(), sin.data_ptr(), rows, d, hd, heads,
                                    ld_dy if ld_dy is not None else d, ld_x if ld_x is not None else d,
                                    ld_dx if ld_dx is not None else d, seq_len, dw_scale, stream_ptr(x.device)),
          "rmsnorm_rope_bwd")
    _count()


def layernorm_fwd(x, w, b, y, mean, rstd, *, rows, d, eps) -> None:
    """y = (x - mean) * rstd * w (+ b) over plain [rows, d] bf16 tensors; w / b may be None; mean / rstd fp32 [rows]."""
    _req_bf16(x, w, b, y)
    check(lib().ob_layernorm_fwd(x.data_ptr(), _ptr(w), _ptr(b), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, d,
                                 eps, stream_ptr(x.device)), "layernorm_fwd")
    _count()


def layernorm_bwd(dy, x, w, mean, rstd, dx, *, rows, d, dw=None, db=None, scale=1.0) -> None:
    _req_bf16(dy, x, w, dx)
    check(lib().ob_layernorm_bwd(dy.data_ptr(), x.data_ptr(), _ptr(w), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                 _ptr(dw), _ptr(db), rows, d, scale, stream_ptr(x.device)), "layernorm_bwd")
    _count()


def rope(x, y, cos, sin, *, sign=1.0, pos_offset=0) -> None:
    """x, y: [B, S, H, D] bf16 (head dim contiguous); cos/sin fp32 [>= S, D/2]."""
    _req_bf16(x, y)
    B, S, H, D = x.shape
    check(lib().ob_rope(x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, S, H, D, x.stride(0), x.stride(1),
                        x.stride(2), y.stride(0), y.stride(1), y.stride(2), sign, pos_offset, stream_ptr(x.device)), "rope")
    _count()


def glu_fwd(g, u, a, gelu: bool) -> None:
    _req_bf16(g, u, a)
    check(lib().ob_glu_fwd(g.data_ptr(), u.data_ptr(), a.data_ptr(), g.numel(), int(gelu), stream_ptr(g.device)), "glu_fwd")
    _count()


def glu_bwd(g, u, da, dg, du, a_out, gelu: bool) -> None:
    _req_bf16(g, u, da, dg, du, a_out)
    check(lib().ob_glu_bwd(g.data_ptr(), u.data_ptr(), da.data_ptr(), dg.data_ptr(), du.data_ptr(), _ptr(a_out), g.numel(),
                           int(gelu), stream_ptr(g.device)), "glu_bwd")
    _count()


def embed_gather(ids, shard_ptrs, rows_per_shard, n_shards, out, d, scale=1.0) -> None:
    check(lib().ob_embed_gather(ids.data_ptr(), shard_ptrs.data_ptr(), rows_per_shard, n_shards, out.data_ptr(),
                                ids.numel(), d, scale, stream_ptr(out.device)), "embed_gather")
    _count()


def embed_scatter(ids, grad_ptrs, rows_per_shard, n_shards, dout, d, scale=1.0) -> None:
    check(lib().ob_embed_scatter(ids.data_ptr(), grad_ptrs.data_ptr(), rows_per_shard, n_shards, dout.data_ptr(),
                                 ids.numel(), d, scale, stream_ptr(dout.device)), "embed_scatter")
    _count()


def ce_fwd_bwd(logits, labels, dlogits, stats, inv_count, *, V, ignore_index=-100, softcap=0.0, z_loss=0.0,
               grad_scale=1.0, lse=None) -> None:
    rows = logits.shape[0]
    check(lib().ob_ce_fwd_bwd(logits.data_ptr(), logits.stride(0), labels.data_ptr(), _ptr(dlogits),
                              dlogits.stride(0) if dlogits is not None else 0, _ptr(lse), stats.data_ptr(),
                              inv_count.data_ptr(), rows, V, ignore_index, softcap, z_loss, grad_scale,
                              stream_ptr(logits.device)), "ce_fwd_bwd")
    _count()


def ce_vp_stats(logits, labels, stats, *, V, vocab_offset, softcap=0.0) -> None:
    """Per-row (max, sum exp, target logit) of this rank's vocabulary slice ``logits [rows, V]`` -> ``stats [rows, 4]``."""
    check(lib().ob_ce_vp_stats(logits.data_ptr(), logits.stride(0), labels.data_ptr(), stats.data_ptr(), logits.shape[0], V,
                               vocab_offset, softcap, stream_ptr(logits.device)), "ce_vp_stats")
    _count()


def ce_vp_grad(logits, labels, dlogits, peer_stats, n_peers, inv_counts, loss_sums, *, V, vocab_offset, V_total,
               rows_per_src, row0, my_src, ignore_index=-100, softcap=0.0, z_loss=0.0, grad_scale=1.0) -> None:
    """Combine the members' statistics (``peer_stats``: device pointer table) and write the gradient of the local logits."""
    check(lib().ob_ce_vp_grad(logits.data_ptr(), logits.stride(0), labels.data_ptr(), _ptr(dlogits),
                              dlogits.stride(0) if dlogits is not None else 0, peer_stats.data_ptr(), n_peers,
                              inv_counts.data_ptr(), rows_per_src, row0, my_src, loss_sums.data_ptr(), logits.shape[0], V,
                              vocab_offset, V_total, ignore_index, softcap, z_loss, grad_scale, stream_ptr(logits.device)),
          "ce_vp_grad")
    _count()


def count_valid(labels, ignore_index, V, out, counter) -> None:
    check(lib().ob_count_valid(labels.data_ptr(), labels.numel(), ignore_index, V, out.data_ptr(), counter.data_ptr(),
                               stream_ptr(labels.device)), "count_valid")
    _count()


def adamw(p, m, v, g, shadow, *, lr, b1, b2, eps, wd, bias_corr1, bias_corr2, gscale=None, zero_grad=False) -> None:
    check(lib().ob_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _ptr(shadow), p.numel(), lr, b1, b2, eps,
                         wd, bias_corr1, bias_corr2, _ptr(gscale), int(zero_grad), stream_ptr(p.device)), "adamw")
    _count()


def sumsq(x, out) -> None:
    check(lib().ob_sumsq(x.data_ptr(), x.numel(), out.data_ptr(), stream_ptr(x.device)), "sumsq")
    _count()


def clip_coef(sumsq_t, max_norm, pre_scale, out) -> None:
    check(lib().ob_clip_coef(sumsq_t.data_ptr(), max_norm, pre_scale, out.data_ptr(), stream_ptr(out.device)), "clip_coef")
    _count()


def cast_f32_bf16(src, dst) -> None:
    check(lib().ob_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), stream_ptr(src.device)), "cast")
    _count()


def gather_shards(table, dst, stride, n_per_shard, n_shards, skip) -> None:
    """dst[r * stride + i] = shard_r[i] for every r != skip; ``table``: device array of shard base pointers."""
    check(lib().ob_gather_shards(table.data_ptr(), dst.data_ptr(), stride, n_per_shard, n_shards, skip,
                                 stream_ptr(dst.device)), "gather_shards")
    _count()


def scatter_add_shards(src, table, n_per_shard, n_shards, scale=1.0) -> None:
    """shard_r[i] += scale * src[r * n_per_shard + i] (fp32 red.add; shards may live on peer GPUs)."""
    check(lib().ob_scatter_add_shards(src.data_ptr(), table.data_ptr(), n_per_shard, n_shards, scale,
                                      stream_ptr(src.device)), "scatter_add_shards")
    _count()


def allreduce_p2p(table, n, me, world, scale=1.0, max_blocks=0) -> None:
    """In-place sum of an fp32 buffer over the GPUs whose buffer addresses are in ``table`` (device pointer array)."""
    check(lib().ob_allreduce_p2p_f32(table.data_ptr(), n, me, world, scale, max_blocks, stream_ptr(table.device)),
          "allreduce_p2p")
    _count()


def allreduce_multimem(mc_ptr: int, n, me, world, max_blocks=0, device=None) -> None:
    """In-place sum through an NVLS multicast address (multimem.ld_reduce / multimem.st)."""
    check(lib().ob_allreduce_multimem_f32(mc_ptr, n, me, world, max_blocks, stream_ptr(device)), "allreduce_multimem")
    _count()


def peer_barrier(table, me: int, n: int, epoch: int, timeout_s: float = 0.0) -> None:
    """Stream-ordered barrier over peer memory (``csrc/comm.h``); a peer that never arrives costs ``timeout_s`` and a
    :class:`KernelError` at the next ``check_status``, not a hang."""
    dev = table.device
    check(lib().ob_peer_barrier(table.data_ptr(), me, n, epoch & 0xFFFFFFFF, int(timeout_s * 1e9),
                                status_buffer(dev).data_ptr(), stream_ptr(dev)), "peer_barrier")
    _count()


def peer_signal(table, me: int, n: int, epoch: int) -> None:
    """First half of :func:`peer_barrier`: publish ``epoch`` to every member (after a system-scope fence)."""
    check(lib().ob_peer_signal(table.data_ptr(), me, n, epoch & 0xFFFFFFFF, stream_ptr(table.device)), "peer_signal")
    _count()


def peer_wait(table, me: int, n: int, epoch: int, timeout_s: float = 0.0) -> None:
    """Second half of :func:`peer_barrier`: wait (bounded) until every member has published ``epoch`` or a later one."""
    dev = table.device
    check(lib().ob_peer_wait(table.data_ptr(), me, n, epoch & 0xFFFFFFFF, int(timeout_s * 1e9),
                             status_buffer(dev).data_ptr(), stream_ptr(dev)), "peer_wait")
    _count()


def copy_bytes(dst_ptr: int, src_ptr: int, nbytes: int, device, blocks: int = 0, unroll: int = 8) -> None:
    """Raw copy between two addresses (either may be peer memory) with our copy kernel."""
    check(lib().ob_copy_bytes(dst_ptr, src_ptr, nbytes, blocks, unroll, stream_ptr(device)), "copy_bytes")
    _count()


def push_copy(table, src, nbytes: int, n_dst: int, skip: int = -1, blocks: int = 0) -> None:
    """dsts[s][:nbytes] = src for every s != skip; ``table``: device array of destination addresses (peers allowed)."""
    check(lib().ob_push_copy(table.data_ptr(), src.data_ptr(), nbytes, n_dst, skip, blocks, stream_ptr(src.device)), "push_copy")
    _count()


def fold_slots_bf16(out, stage, n, slots, slot_stride, *, skip=-1, accumulate=False) -> None:
    """out[:n] = (out if accumulate) + sum over slots r != skip of stage[r * slot_stride : ... + n]  (bf16, fp32 sums)."""
    _req_bf16(out, stage)
    check(lib().ob_fold_slots_bf16(out.data_ptr(), stage.data_ptr(), n, slots, slot_stride, skip, int(accumulate),
                                   stream_ptr(out.device)), "fold_slots_bf16")
    _count()


def reduce_slots(stage, acc, n, R, slot_stride, scale=1.0) -> None:
    """acc[:n] += scale * sum_r stage[r * slot_stride : r * slot_stride + n] (fp32 accumulator; fp32 or bf16 slots)."""
    fn = lib().ob_reduce_slots_bf16 if stage.dtype == torch.bfloat16 else lib().ob_reduce_slots_f32
    check(fn(stage.data_ptr(), acc.data_ptr(), n, R, slot_stride, scale, stream_ptr(acc.device)), "reduce_slots")
    _count()


# ----------------------------------------------------------------------------------------------------------------------
# Optional per-kernel device timing (OLMAX_B200_KERNEL_TIMING=1): every wrapper above is bracketed by CUDA events on
# the launching stream; `timing_report()` synchronises and sums them per label.  Events add a few microseconds of
# host time per launch, so this is a profiling mode, not something to leave on for a measured run.
# ----------------------------------------------------------------------------------------------------------------------
_TIMED: list = []
_TIMING_ON = os.environ.get("OLMAX_B200_KERNEL_TIMING", "0") == "1"


def timing_enabled() -> bool:
    return _TIMING_ON


def set_timing(on: bool) -> None:
    global _TIMING_ON
    _TIMING_ON = bool(on)
    _TIMED.clear()


@contextlib.contextmanager
def timed_region(label: str):
    """Device time of everything enqueued on the current stream inside the block (collectives, copies, ...)."""
    if not _TIMING_ON or not torch.cuda.is_available():
        yield
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    try:
        yield
    finally:
        e1.record()
        _TIMED.append((label, e0, e1))


def _gemm_label(args, kwargs) -> str:
    M, N, Kd = args[3], args[4], args[5]
    tags = []
    if kwargs.get("a_mn"):
        tags.append("A^T")
    if kwargs.get("b_mn"):
        tags.append("B^T")
    epi = kwargs.get("epi", EPI_BF16)
    tags.append(["bf16", "f32", "f32+=", "f32red", "swiglu", "geglu", "bf16+="][epi])
    if kwargs.get("ag_src") is not None:
        tags.append("AG(A)" if kwargs.get("ag_on_a") else "AG(B)")
    if kwargs.get("c_shards") is not None:
        tags.append("RS")
    if kwargs.get("prefetch") is not None:
        tags.append("pf")
    return f"gemm {M}x{N}x{Kd} " + " ".join(tags)


def _timed(name: str, fn):
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if not _TIMING_ON:
            return fn(*args, **kwargs)
        label = _gemm_label(args, kwargs) if name == "gemm" else name
        with timed_region(label):
            return fn(*args, **kwargs)

    return wrapper


def timing_report(reset: bool = True) -> dict:
    """{label: (launches, total device ms)} of the launches recorded since the last reset."""
    if not _TIMED:
        return {}
    torch.cuda.synchronize()
    out: dict = {}
    for label, e0, e1 in _TIMED:
        n, ms = out.get(label, (0, 0.0))
        out[label] = (n + 1, ms + e0.elapsed_time(e1))
    if reset:
        _TIMED.clear()
    return out


def format_timing(report: dict, top: int = 40) -> str:
    total = sum(ms for _, ms in report.values()) or 1.0
    rows = sorted(report.items(), key=lambda kv: -kv[1][1])[:top]
    lines = [f"{'label':58s} {'n':>6s} {'ms':>10s} {'share':>7s}"]
    for label, (n, ms) in rows:
        lines.append(f"{label[:58]:58s} {n:6d} {ms:10.3f} {100 * ms / total:6.1f}%")
    lines.append(f"{'sum of timed regions':58s} {'':6s} {total:10.3f}")
    return "\n".join(lines)


for _name in ("gemm", "flash_attn_fwd", "flash_attn_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "rmsnorm_rope_fwd",
              "rmsnorm_rope_bwd", "layernorm_fwd", "layernorm_bwd",
              "rope", "glu_fwd", "glu_bwd", "embed_gather", "embed_scatter", "ce_fwd_bwd", "ce_vp_stats", "ce_vp_grad", "count_valid",
              "adamw", "sumsq",
              "clip_coef", "cast_f32_bf16", "gather_shards", "scatter_add_shards", "allreduce_p2p", "allreduce_multimem",
              "copy_bytes", "push_copy", "fold_slots_bf16", "reduce_slots", "peer_barrier", "peer_signal", "peer_wait"):
    globals()[_name] = _timed(_name, globals()[_name])

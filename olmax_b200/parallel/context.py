"""
Context parallelism: the sequence dimension of every activation is split over the mesh's CP axis and causal attention
runs across the ranks of that axis (role of the TransformerEngine path of ``olmax/nn/attention.py:64-94`` and the
re-ordering helpers of ``olmax/distributed/parallel.py:381-394``).

Token placement ("dual chunk swap"): a sequence of length S is cut into ``2 * cp`` chunks of ``c = S / (2 cp)``
tokens and rank r holds chunk r followed by chunk ``2 cp - 1 - r``, which gives every rank the same amount of causal
work.  Inputs, labels and the RoPE tables are re-ordered the same way.

Two strategies, both built from the rectangular flash-attention kernels (a query block at key-axis offset ``q_off``
against a key block; forward returns the row log-sum-exp, backward takes the row statistics of the whole softmax):

* ``all_gather``: K and V are gathered over the CP axis into natural order; each of the two local query chunks
  attends to the prefix of the sequence that is causally visible to it (trimmed on the left to the sliding window);
  backward reduce-scatters the fp32 dK / dV.
* ``ring``: K / V blocks travel around the ring (``cp`` steps, the transfer of step t+1 is posted before the math of
  step t); a rank attends to the visiting block with whichever of its two query chunks can see it and merges the
  partial outputs with their log-sum-exps; in backward the dK / dV accumulators travel with their block and arrive
  home after ``cp`` hops.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..types import StrEnum
from . import collectives as coll

__all__ = [
    "CPStrategy",
    "cp_local_positions",
    "reorder_causal_load_balancing",
    "inverse_reorder_causal_load_balancing",
    "shard_sequence_for_cp",
    "context_parallel_attention",
]


class CPStrategy(StrEnum):
    default = "default"        # all_gather
    all_gather = "all_gather"
    ring = "ring"


def _chunk_order(cp_size: int) -> List[int]:
    order: List[int] = []
    for r in range(cp_size):
        order += [r, 2 * cp_size - 1 - r]
    return order


def reorder_causal_load_balancing(x: torch.Tensor, cp_size: int, seq_dim: int) -> torch.Tensor:
    """Natural order -> dual-chunk-swap order along ``seq_dim`` (slice r of ``cp_size`` equal slices is rank r's)."""
    if cp_size == 1:
        return x
    S = x.shape[seq_dim]
    if S % (2 * cp_size):
        raise ValueError(f"sequence length {S} must be a multiple of 2 * cp = {2 * cp_size}")
    chunks = x.chunk(2 * cp_size, dim=seq_dim)
    return torch.cat([chunks[i] for i in _chunk_order(cp_size)], dim=seq_dim)


def inverse_reorder_causal_load_balancing(x: torch.Tensor, cp_size: int, seq_dim: int) -> torch.Tensor:
    if cp_size == 1:
        return x
    chunks = x.chunk(2 * cp_size, dim=seq_dim)
    order = _chunk_order(cp_size)
    out: List[Optional[torch.Tensor]] = [None] * (2 * cp_size)
    for pos, idx in enumerate(order):
        out[idx] = chunks[pos]
    return torch.cat(out, dim=seq_dim)  # type: ignore[arg-type]


def cp_local_positions(seq_len: int, cp_size: int, cp_rank: int, device=None) -> torch.Tensor:
    """Positions (in the full sequence) of the tokens rank ``cp_rank`` holds, in the order it holds them."""
    if cp_size == 1:
        return torch.arange(seq_len, device=device)
    c = seq_len // (2 * cp_size)
    a, b = cp_rank, 2 * cp_size - 1 - cp_rank
    return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])


def shard_sequence_for_cp(x: torch.Tensor, cp_size: int, cp_rank: int, seq_dim: int = 1) -> torch.Tensor:
    """This rank's tokens of a ``[..., S, ...]`` tensor in natural order (inputs, labels)."""
    if cp_size == 1:
        return x
    pos = cp_local_positions(x.shape[seq_dim], cp_size, cp_rank, device=x.device)
    return x.index_select(seq_dim, pos).contiguous()


# ----------------------------------------------------------------------------------------------------------------------
def _block_ops():
    from ..ops import functional as F   # imported late: ops imports parallel

    return F.attention_block_fwd, F.attention_block_bwd


def _align_down(x: int, a: int = 128) -> int:
    return (x // a) * a


def _gather_natural(local: torch.Tensor, group) -> torch.Tensor:
    """local [B, 2c, h, D] (chunk r | chunk 2cp-1-r) on every rank -> [B, S, h, D] in natural order."""
    cp = group.size
    B, two_c = local.shape[0], local.shape[1]
    c = two_c // 2
    buf = torch.empty((cp,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    coll.all_gather_into(buf, local.contiguous(), group)
    full = torch.empty((B, 2 * cp * c) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    for r in range(cp):
        full[:, r * c : (r + 1) * c] = buf[r][:, :c]
        full[:, (2 * cp - 1 - r) * c : (2 * cp - r) * c] = buf[r][:, c:]
    return full


def _scatter_natural(full: torch.Tensor, group) -> torch.Tensor:
    """Sum ``full`` [B, S, h, D] (natural order) over the group and return this rank's [B, 2c, h, D] slice."""
    cp = group.size
    B, S = full.shape[0], full.shape[1]
    c = S // (2 * cp)
    buf = torch.empty((cp, B, 2 * c) + tuple(full.shape[2:]), dtype=full.dtype, device=full.device)
    for r in range(cp):
        buf[r][:, :c] = full[:, r * c : (r + 1) * c]
        buf[r][:, c:] = full[:, (2 * cp - 1 - r) * c : (2 * cp - r) * c]
    out = torch.empty((B, 2 * c) + tuple(full.shape[2:]), dtype=full.dtype, device=full.device)
    coll.reduce_scatter_into(out, buf, group, predivide=False)
    return out


class _AllGatherCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, window, softcap, scale):
        fwd, _ = _block_ops()
        cp, r = group.size, group.rank
        c = q.shape[1] // 2
        kf, vf = _gather_natural(k, group), _gather_natural(v, group)
        o = torch.empty_like(q)
        lse = torch.empty((q.shape[0], q.shape[2], 2 * c), dtype=torch.float32, device=q.device)
        spans = []
        for half, chunk in enumerate((r, 2 * cp - 1 - r)):
            pos0, end = chunk * c, (chunk + 1) * c
            k0 = _align_down(max(0, pos0 - window)) if window >= 0 else 0
            oo, ll = fwd(q[:, half * c : (half + 1) * c], kf[:, k0:end], vf[:, k0:end], q_off=pos0 - k0, causal=True,
                         window=window, softcap=softcap, scale=scale)
            o[:, half * c : (half + 1) * c] = oo
            lse[:, :, half * c : (half + 1) * c] = ll
            spans.append((k0, end, pos0 - k0))
        ctx.group, ctx.cfg, ctx.spans = group, (window, softcap, scale), spans
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, d_o):
        _, bwd = _block_ops()
        q, k, v, o, lse = ctx.saved_tensors
        group = ctx.group
        window, softcap, scale = ctx.cfg
        c = q.shape[1] // 2
        kf, vf = _gather_natural(k, group), _gather_natural(v, group)
        dq = torch.empty_like(q)
        dkf = torch.zeros(kf.shape, dtype=torch.float32, device=q.device)
        dvf = torch.zeros(vf.shape, dtype=torch.float32, device=q.device)
        d_o = d_o.contiguous()
        for half, (k0, end, q_off) in enumerate(ctx.spans):
            sl = slice(half * c, (half + 1) * c)
            g = bwd(q[:, sl], kf[:, k0:end], vf[:, k0:end], o[:, sl], lse[:, :, sl].contiguous(), d_o[:, sl],
                    q_off=q_off, causal=True, window=window, softcap=softcap, scale=scale)
            dq[:, sl] = g[0]
            dkf[:, k0:end] += g[1]
            dvf[:, k0:end] += g[2]
        dk = _scatter_natural(dkf, group).to(k.dtype)
        dv = _scatter_natural(dvf, group).to(v.dtype)
        return dq, dk, dv, None, None, None, None


def _ring_exchange(send: torch.Tensor, recv: torch.Tensor, group):
    """Post send-to-next / receive-from-previous on the CP ring; returns the requests to wait on."""
    nxt = group.ranks[(group.rank + 1) % group.size]
    prv = group.ranks[(group.rank - 1) % group.size]
    ops = [dist.P2POp(dist.isend, send, nxt, group=group.pg), dist.P2POp(dist.irecv, recv, prv, group=group.pg)]
    return dist.batch_isend_irecv(ops)


def _ring_pairs(r: int, j: int, cp: int) -> List[Tuple[int, int, int]]:
    """(query half, key half, chunk distance) for the block pairs rank r computes while it holds rank j's K/V:
    halves index the (chunk x | chunk 2cp-1-x) layout, distance = query chunk - key chunk >= 0 (0: the diagonal)."""
    pairs = [(1, 0, (2 * cp - 1 - r) - j)]          # late query chunk sees every early key chunk
    if j <= r:
        pairs.append((0, 0, r - j))                 # early query chunk vs early key chunk
    if j >= r:
        pairs.append((1, 1, j - r))                 # late query chunk vs late key chunk
    return pairs


def _merge(o_acc, lse_acc, o_new, lse_new):
    """Fold a partial softmax (o_new, lse_new) into the running (o_acc fp32 [B,S,H,D], lse_acc [B,H,S])."""
    lse = torch.logaddexp(lse_acc, lse_new)
    w_old = torch.exp(lse_acc - lse).permute(0, 2, 1).unsqueeze(-1)
    w_new = torch.exp(lse_new - lse).permute(0, 2, 1).unsqueeze(-1)
    return o_acc * w_old + o_new.float() * w_new, lse


class _RingCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, softcap, scale):
        fwd, _ = _block_ops()
        cp, r = group.size, group.rank
        B, two_c, H, D = q.shape
        c = two_c // 2
        kv = torch.stack((k, v)).contiguous()
        o_acc = torch.zeros((B, two_c, H, D), dtype=torch.float32, device=q.device)
        lse_acc = torch.full((B, H, two_c), float("-inf"), dtype=torch.float32, device=q.device)
        for t in range(cp):
            j = (r - t) % cp
            nxt_kv, reqs = None, []
            if t + 1 < cp:
                nxt_kv = torch.empty_like(kv)
                reqs = _ring_exchange(kv, nxt_kv, group)
            for qh, kh, dist_c in _ring_pairs(r, j, cp):
                qs, ks = slice(qh * c, (qh + 1) * c), slice(kh * c, (kh + 1) * c)
                oo, ll = fwd(q[:, qs], kv[0][:, ks], kv[1][:, ks], q_off=dist_c * c, causal=True, window=-1,
                             softcap=softcap, scale=scale)
                o_acc[:, qs], lse_acc[:, :, qs] = _merge(o_acc[:, qs], lse_acc[:, :, qs], oo, ll)
            for req in reqs:
                req.wait()
            if nxt_kv is not None:
                kv = nxt_kv
        o = o_acc.to(q.dtype)
        ctx.group, ctx.cfg = group, (softcap, scale)
        ctx.save_for_backward(q, k, v, o, lse_acc)
        return o

    @staticmethod
    def backward(ctx, d_o):
        _, bwd = _block_ops()
        q, k, v, o, lse = ctx.saved_tensors
        group = ctx.group
        softcap, scale = ctx.cfg
        cp, r = group.size, group.rank
        c = q.shape[1] // 2
        d_o = d_o.contiguous()
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)   # travels with its K/V block
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for t in range(cp):
            j = (r - t) % cp
            nxt_kv, reqs = None, []
            if t + 1 < cp:
                nxt_kv = torch.empty_like(kv)
                reqs = _ring_exchange(kv, nxt_kv, group)
            for qh, kh, dist_c in _ring_pairs(r, j, cp):
                qs, ks = slice(qh * c, (qh + 1) * c), slice(kh * c, (kh + 1) * c)
                g = bwd(q[:, qs], kv[0][:, ks], kv[1][:, ks], o[:, qs], lse[:, :, qs].contiguous(), d_o[:, qs],
                        q_off=dist_c * c, causal=True, window=-1, softcap=softcap, scale=scale)
                dq[:, qs] += g[0]
                dkv[0][:, ks] += g[1]
                dkv[1][:, ks] += g[2]
            for req in reqs:
                req.wait()
            # the accumulator follows its block: after the last step one more hop brings it home
            nxt_dkv = torch.empty_like(dkv)
            for req in _ring_exchange(dkv, nxt_dkv, group):
                req.wait()
            dkv = nxt_dkv
            if nxt_kv is not None:
                kv = nxt_kv
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def context_parallel_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, *,
                               strategy: CPStrategy = CPStrategy.default, window: int = -1, softcap: float = 0.0,
                               scale: Optional[float] = None) -> torch.Tensor:
    """
    Causal attention over a sequence split across ``group`` in dual-chunk-swap order.  q [B, S/cp, H, D],
    k / v [B, S/cp, Hkv, D] hold this rank's two chunks; returns this rank's rows of the output.  A sliding window
    narrower than the sequence is handled by the all-gather strategy (the ring strategy falls back to it).
    """
    if q.shape[1] % 2:
        raise ValueError("context parallelism needs an even number of local tokens (two chunks per rank)")
    window = -1 if window is None else int(window)
    strategy = CPStrategy(strategy)
    S = q.shape[1] * group.size
    if strategy == CPStrategy.ring and (window < 0 or window >= S - 1):
        return _RingCPAttention.apply(q, k, v, group, softcap or 0.0, scale)
    return _AllGatherCPAttention.apply(q, k, v, group, window, softcap or 0.0, scale)

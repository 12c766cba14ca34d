"""
Multi-head self-attention (``olmax/nn/attention.py:1-376``): separate q/k/v/o projections, optional QK-norm (over the
full projection or per head), RoPE on q and k, causal flash attention with grouped KV heads, optional sliding window
and logit soft-cap.  Under tensor parallelism the heads are split over the TP axis (q/k/v colwise, o rowwise) and the
block runs between a sequence all-gather and a sequence reduce-scatter.  Under context parallelism every rank holds
two chunks of each sequence (``parallel/context.py``): RoPE uses the chunks' positions and the attention kernel is
replaced by the all-gather or ring composition of rectangular flash-attention blocks.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops import functional as F
from ..parallel import collectives as coll
from ..parallel.context import CPStrategy, context_parallel_attention
from ..parallel.mesh import TPStyle
from ..types import StrEnum
from .linear import Linear
from .module import Module, current_build_context
from .normalization import NormalizerConfig, RMSNorm, RMSNormConfig
from .rope import BufferCache, RotaryPositionalEmbedding, RotaryPositionalEmbeddingConfig

__all__ = ["AttentionImplementation", "AttentionKernel", "MultiheadSelfAttention", "MultiheadSelfAttentionConfig"]


class AttentionImplementation(StrEnum):
    """``flash_sm100`` is the hand-written kernel (CUDA) / the PyTorch restatement (CPU).  The reference's names are
    accepted as aliases so that its configs parse."""

    flash_sm100 = "flash_sm100"
    xla = "xla"
    cudnn = "cudnn"
    te_fused = "te_fused"


class AttentionKernel(torch.nn.Module):
    """Scaled-dot-product attention on ``[B, S, H, D]`` tensors (``olmax/nn/attention.py:23-109``)."""

    def __init__(self, head_dim: int, window_size: Optional[int] = None, logit_softcap: Optional[float] = None,
                 implementation: Optional[AttentionImplementation] = None, cp_strategy: Optional[str] = None,
                 cp_group=None):
        super().__init__()
        self.head_dim = head_dim
        self.window_size = window_size
        self.logit_softcap = logit_softcap
        self.implementation = AttentionImplementation.flash_sm100
        self.cp_strategy = CPStrategy(cp_strategy) if cp_strategy is not None else CPStrategy.default
        self.cp_group = cp_group
        self.scale = 1.0 / math.sqrt(head_dim)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        window = self.window_size if self.window_size is not None else -1
        if self.cp_group is not None and self.cp_group.size > 1:
            return context_parallel_attention(q, k, v, self.cp_group, strategy=self.cp_strategy, window=window,
                                              softcap=self.logit_softcap or 0.0, scale=self.scale)
        return F.attention(q, k, v, causal=True, window=window, softcap=self.logit_softcap or 0.0, scale=self.scale)


class MultiheadSelfAttention(Module):
    def __init__(
        self,
        d_model: int,
        n_heads: int,
        n_kv_heads: Optional[int] = None,
        head_dim: Optional[int] = None,
        bias: bool = False,
        rope: Optional[RotaryPositionalEmbeddingConfig] = None,
        qk_norm: Optional[NormalizerConfig] = None,
        use_head_qk_norm: bool = False,
        window_size: Optional[int] = None,
        logit_softcap: Optional[float] = None,
        init_std: float = 0.02,
        cp_strategy: Optional[str] = None,
    ):
        super().__init__()
        ctx = current_build_context()
        self.d_model = d_model
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.head_dim = head_dim or d_model // n_heads
        tp = self.mesh.tp.size
        if tp > 1 and self.mesh.cp.size > 1:
            raise ValueError("tensor parallelism and context parallelism cannot be combined")
        if self.n_heads % tp or self.n_kv_heads % tp:
            raise ValueError(f"heads ({self.n_heads}/{self.n_kv_heads}) must be divisible by the TP degree {tp}")
        self.local_heads = self.n_heads // tp
        self.local_kv_heads = self.n_kv_heads // tp
        self.use_head_qk_norm = use_head_qk_norm
        with ctx.scope("q_proj"):
            self.q_proj = Linear(d_model, self.n_heads * self.head_dim, bias=bias, tp_style=TPStyle.colwise, init_std=init_std)
        with ctx.scope("k_proj"):
            self.k_proj = Linear(d_model, self.n_kv_heads * self.head_dim, bias=bias, tp_style=TPStyle.colwise, init_std=init_std)
        with ctx.scope("v_proj"):
            self.v_proj = Linear(d_model, self.n_kv_heads * self.head_dim, bias=bias, tp_style=TPStyle.colwise, init_std=init_std)
        with ctx.scope("o_proj"):
            self.o_proj = Linear(self.n_heads * self.head_dim, d_model, bias=bias, tp_style=TPStyle.rowwise, init_std=init_std)
        self.q_norm = self.k_norm = None
        if qk_norm is not None:
            if tp > 1 and not use_head_qk_norm:
                raise ValueError("QK-norm over the full projection is not compatible with head-split tensor parallelism")
            # the full-projection k-norm has n_kv_heads * head_dim entries (the reference sizes it with n_heads,
            # which only works without GQA, olmax/nn/attention.py:248-249)
            qn = self.head_dim if use_head_qk_norm else self.n_heads * self.head_dim
            kn = self.head_dim if use_head_qk_norm else self.n_kv_heads * self.head_dim
            with ctx.scope("q_norm"):
                self.q_norm = qk_norm.build(qn)
            with ctx.scope("k_norm"):
                self.k_norm = qk_norm.build(kn)
        self.rope = rope.build(self.head_dim) if rope is not None else None
        self.recompute = False
        """Set by the layer when the activation-checkpointing policy recomputes this block: q / k / v are rebuilt in the
        block's own backward node instead of being kept (``ops/functional.py: recomputed_attention``)."""
        self.sdpa = AttentionKernel(self.head_dim, window_size=window_size, logit_softcap=logit_softcap,
                                    cp_strategy=cp_strategy, cp_group=self.mesh.cp)

    def _qkv(self, x: torch.Tensor, batch_size: int, cache: Optional[BufferCache]):
        """Block input -> (q [B,S,H,D], k, v [B,S,Hkv,D]): projections, q / k norm, rotation."""
        tp = self.mesh.tp
        tpc = self.store.tp_symm if x.is_cuda else None
        if tpc is not None:
            # the all-gather of x over the TP group is fused into the q GEMM (k and v read the gathered rows)
            q, k, v = F.tp_column_linears(x, tpc, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
        else:
            x = coll.seq_all_gather(x, tp)
            q = self.q_proj(x)
            k = self.k_proj(x)
            v = self.v_proj(x)
        T = q.shape[0]
        S = T // batch_size
        heads_q = self.local_heads if self.use_head_qk_norm else 1
        heads_k = self.local_kv_heads if self.use_head_qk_norm else 1
        v = v.view(batch_size, S, self.local_kv_heads, self.head_dim)
        if isinstance(self.q_norm, RMSNorm) and self.rope is not None:
            # q / k normalisation and the rotary embedding in one pass over each projection
            cp = self.mesh.cp
            cos, sin = self.rope.tables_for(S, x.device, cache, cp.size, cp.rank)
            q = F.rms_norm_rope(q, self.q_norm.weight, self.q_norm.eps, heads_q, cos, sin, batch_size, self.head_dim)
            k = F.rms_norm_rope(k, self.k_norm.weight, self.k_norm.eps, heads_k, cos, sin, batch_size, self.head_dim)
        else:
            if self.q_norm is not None:
                q = self.q_norm(q, heads=heads_q)
                k = self.k_norm(k, heads=heads_k)
            q = q.view(batch_size, S, self.local_heads, self.head_dim)
            k = k.view(batch_size, S, self.local_kv_heads, self.head_dim)
            if self.rope is not None:
                cp = self.mesh.cp
                q = self.rope(q, cache, cp.size, cp.rank)
                k = self.rope(k, cache, cp.size, cp.rank)
        return q, k, v

    @property
    def recomputes_itself(self) -> bool:
        """True when the block can drop q / k / v after the forward pass and rebuild them in its own backward node
        (not under context parallelism, whose attention is a composition of block kernels with its own backward)."""
        return self.mesh.cp.size == 1

    def forward(self, x: torch.Tensor, batch_size: int, cache: Optional[BufferCache] = None) -> torch.Tensor:
        """x: [tokens, d_model] (tokens = batch * seq, or that divided by tp under sequence parallelism)."""
        tp = self.mesh.tp
        tpc = self.store.tp_symm if x.is_cuda else None
        if self.recompute and self.recomputes_itself and torch.is_grad_enabled() and x.requires_grad:
            k = self.sdpa
            o = F.recomputed_attention(x, lambda t: self._qkv(t, batch_size, cache),
                                       k.window_size if k.window_size is not None else -1, k.logit_softcap or 0.0, k.scale)
        else:
            o = self.sdpa(*self._qkv(x, batch_size, cache))
        o = o.reshape(-1, self.local_heads * self.head_dim)
        if tpc is not None:
            return F.tp_row_linear(o, tpc, self.o_proj.weight)   # reduce-scatter fused into the GEMM epilogue
        y = self.o_proj(o)
        return coll.seq_reduce_scatter(y, tp)


@dataclass
class MultiheadSelfAttentionConfig:
    n_heads: int = 16
    n_kv_heads: Optional[int] = None
    head_dim: Optional[int] = None
    bias: bool = False
    rope: Optional[RotaryPositionalEmbeddingConfig] = field(default_factory=RotaryPositionalEmbeddingConfig)
    qk_norm: Optional[NormalizerConfig] = None
    use_head_qk_norm: bool = False
    window_size: Optional[int] = None
    logit_softcap: Optional[float] = None
    implementation: Optional[AttentionImplementation] = None
    cp_strategy: Optional[str] = None
    """``default`` / ``all_gather`` / ``ring`` (``olmax/nn/attention.py:29``); only read on a mesh with a CP axis."""

    def build(self, d_model: int, window_size: Optional[int] = "inherit", init_std: float = 0.02) -> MultiheadSelfAttention:
        return MultiheadSelfAttention(
            d_model, self.n_heads, self.n_kv_heads, self.head_dim, self.bias, self.rope, self.qk_norm,
            self.use_head_qk_norm, self.window_size if window_size == "inherit" else window_size, self.logit_softcap,
            init_std=init_std, cp_strategy=self.cp_strategy,
        )

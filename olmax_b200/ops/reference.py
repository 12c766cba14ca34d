"""
Plain PyTorch restatement of every op's math.  It is the numerical oracle of the CUDA kernels (GPU tests compare a
kernel against these functions evaluated in fp32) and it is the implementation used on CPU, where the multi-process
(gloo) tests and the tiny fp32 configuration run.

Semantics follow the reference: RMSNorm upcasts to fp32, multiplies by ``rsqrt(mean(x^2) + eps)`` and by the weight,
then casts back (``olmax/nn/functional.py:51-67``); RoPE is the rotate-half form computed in fp32
(``olmax/nn/rope.py:99-115``); attention is causal soft-max attention with scale ``1/sqrt(head_dim)``, grouped KV
heads and an optional left window (``olmax/nn/attention.py:96-103``) plus an optional tanh soft-cap; the MLP is
``down(act(gate(x)) * up(x))`` (``olmax/nn/mlp.py:69-73``); cross entropy excludes ``ignore_index`` rows from both
numerator and denominator (``olmax/nn/functional.py:70-121``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "rms_norm", "layer_norm", "rope_tables", "apply_rope", "attention", "glu", "cross_entropy", "fused_cross_entropy",
    "softcap", "activation",
]


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-5,
             bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    dt = x.dtype
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(dt)


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    dt = x.dtype
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(dt)


def rope_tables(seq_len: int, head_dim: int, theta: float, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin of shape [seq_len, head_dim // 2] in fp32: angle = position * theta^(-2i / head_dim)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    pos = torch.arange(seq_len, dtype=torch.float32, device=device)
    ang = torch.outer(pos, inv_freq)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, sign: float = 1.0) -> torch.Tensor:
    """x: [B, S, H, D]; out = x * [cos, cos] + rotate_half(x) * [sin, sin]."""
    dt = x.dtype
    S, D = x.shape[1], x.shape[-1]
    xf = x.float()
    c = cos[:S].view(1, S, 1, D // 2)
    s = sin[:S].view(1, S, 1, D // 2) * sign
    lo, hi = xf[..., : D // 2], xf[..., D // 2 :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(dt)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x / cap) if cap and cap > 0 else x


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, window: int = -1,
              logit_softcap: float = 0.0, scale: Optional[float] = None, q_off: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,S,H,D], k/v [B,Sk,Hkv,D] -> (o [B,S,H,D], lse [B,H,S]).  Query row i sits at position ``q_off + i`` of the
    key axis; window >= 0 keeps keys j >= position - window."""
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = softcap(s, logit_softcap)
    Sk = k.shape[1]
    i = torch.arange(S, device=q.device).view(S, 1) + q_off
    j = torch.arange(Sk, device=q.device).view(1, Sk)
    mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= j <= i
    if window is not None and window >= 0:
        mask &= j >= i - window
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def attention_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                  d_o: torch.Tensor, causal: bool = True, window: int = -1, logit_softcap: float = 0.0,
                  scale: Optional[float] = None, q_off: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of one (query block, key block) pair of a softmax whose row statistics are given: ``lse`` [B,H,S] is
    the log-sum-exp over ALL keys of the row (not only this block's) and ``o`` the final output, so the pieces of a
    blockwise / ring attention add up to the gradient of the whole."""
    B, S, H, D = q.shape
    Hkv, Sk = k.shape[2], k.shape[1]
    G = H // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    dof = d_o.float().permute(0, 2, 1, 3)
    raw = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = softcap(raw, logit_softcap)
    i = torch.arange(S, device=q.device).view(S, 1) + q_off
    j = torch.arange(Sk, device=q.device).view(1, Sk)
    mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= j <= i
    if window is not None and window >= 0:
        mask &= j >= i - window
    p = torch.exp(s - lse.float().unsqueeze(-1)).masked_fill(~mask, 0.0)
    delta = (o.float() * d_o.float()).sum(-1).permute(0, 2, 1).unsqueeze(-1)   # [B,H,S,1]
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta)
    if logit_softcap and logit_softcap > 0:
        ds = ds * (1.0 - torch.tanh(raw / logit_softcap) ** 2)
    ds = ds * scale
    dq = torch.matmul(ds, kf).permute(0, 2, 1, 3)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(B, Hkv, G, Sk, D).sum(2).permute(0, 2, 1, 3)
    dv = dv.view(B, Hkv, G, Sk, D).sum(2).permute(0, 2, 1, 3)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def activation(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "silu":
        return F.silu(x)
    if name in ("gelu", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    raise ValueError(f"unknown activation '{name}'")


def glu(g: torch.Tensor, u: torch.Tensor, act: str = "silu") -> torch.Tensor:
    return (activation(act, g.float()) * u.float()).to(g.dtype)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, reduction: str = "mean",
                  logit_softcap: float = 0.0) -> torch.Tensor:
    loss, _ = fused_cross_entropy(logits, labels, ignore_index=ignore_index, reduction=reduction,
                                  logit_softcap=logit_softcap)
    return loss


def fused_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, reduction: str = "mean",
                        z_loss_multiplier: float = 0.0, logit_softcap: float = 0.0):
    """(loss, z_loss).  Labels outside [0, V) other than ``ignore_index`` contribute zero loss but still count in the
    mean, as a one-hot of an out-of-range class is all zero (``olmax/nn/functional.py:70-91``)."""
    lf = softcap(logits.float(), logit_softcap)
    V = lf.shape[-1]
    lf2 = lf.reshape(-1, V)
    lab = labels.reshape(-1)
    lse = torch.logsumexp(lf2, dim=-1)
    counted = lab != ignore_index
    in_range = counted & (lab >= 0) & (lab < V)
    tgt = lf2.gather(1, lab.clamp(0, V - 1).view(-1, 1)).view(-1)
    per_tok = torch.where(in_range, lse - tgt, torch.zeros_like(lse))
    z = torch.where(counted, lse.pow(2), torch.zeros_like(lse)) * z_loss_multiplier
    if reduction == "mean":
        n = counted.sum().clamp(min=1)
        return per_tok.sum() / n, z.sum() / n
    if reduction == "sum":
        return per_tok.sum(), z.sum()
    return per_tok.view(labels.shape), z.view(labels.shape)

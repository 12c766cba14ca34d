"""
The decoder-only transformer (``olmax/nn/transformer/model.py:1-213``): embedding -> layers -> final norm -> LM head,
built directly into a sharded :class:`ParamStore`.  Each of {embedding, every layer, final norm + head} is one FSDP
unit: its weights are gathered right before use (prefetched one unit ahead), released after use and gathered again
for the backward pass, and its weight gradients are reduce-scattered as soon as its backward has run.
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..activation_checkpointing import ActivationCheckpointingPolicy, NamedCheckpointPolicy, NoPolicy
from ..nn.embedding import Embedding
from ..nn.lm_head import LMHead, LMHeadConfig
from ..nn.module import BuildContext, Module
from ..nn.normalization import NormalizerConfig, RMSNormConfig
from ..nn.rope import BufferCache
from ..parallel import dist_utils
from ..parallel.mesh import DeviceMesh, MeshResource, get_mesh
from ..parallel.param_store import FSDPUnit, ParamStore
from ..utils.dataclass_codec import Registrable
from .layer import DefaultTransformerLayerConfig, TransformerLayerConfig

__all__ = ["Transformer", "TransformerConfig", "DefaultTransformerConfig"]


class _UnitEnter(torch.autograd.Function):
    """Forward: make sure the unit's weights are gathered, prefetch the next unit.  Backward (runs after the unit's
    own backward): reduce-scatter its weight gradients and drop the gathered weights."""

    @staticmethod
    def forward(ctx, x, delta, unit: FSDPUnit):
        ctx.unit = unit
        ctx.has_delta = delta is not None
        unit.start_gather()
        unit.store.prefetch(unit.index + 1)
        if delta is None:
            return x.view_as(x)
        return x.view_as(x), delta.view_as(delta)

    @staticmethod
    def backward(ctx, *grads):
        unit = ctx.unit
        unit.reduce_grads()
        unit.release()
        if ctx.has_delta:
            return grads[0], grads[1], None
        return grads[0], None, None


class _UnitExit(torch.autograd.Function):
    """Forward: release the gathered weights (when resharding after forward).  Backward (runs before the unit's own
    backward): gather them again and prefetch the unit that comes next in the backward order."""

    @staticmethod
    def forward(ctx, x, delta, unit: FSDPUnit):
        ctx.unit = unit
        ctx.has_delta = delta is not None
        if unit.store.reshard_after_forward and unit.store.mesh.shard.size > 1:
            unit.release()
        if delta is None:
            return x.view_as(x)
        return x.view_as(x), delta.view_as(delta)

    @staticmethod
    def backward(ctx, *grads):
        unit = ctx.unit
        unit.store._in_backward = True
        unit.start_gather()
        unit.store.prefetch(unit.index - 1)
        if ctx.has_delta:
            return grads[0], grads[1], None
        return grads[0], None, None


def _enter(x, delta, unit):
    out = _UnitEnter.apply(x, delta, unit)
    return (out, None) if delta is None else out


def _exit(x, delta, unit):
    out = _UnitExit.apply(x, delta, unit)
    return (out, None) if delta is None else out


class Transformer(Module):
    def __init__(self, config: "TransformerConfig"):
        super().__init__()
        ctx = BuildContext(self.store)
        self.config = config
        d = config.d_model
        policy = config.layer_ac_policy or NoPolicy()
        emb_scale = math.sqrt(d) if config.scale_embeddings else 1.0
        with ctx.scope("embedding", unit="embedding"):
            self.embedding = Embedding(config.vocab_size, d, scale=emb_scale, init_std=config.init_std)
        layers = []
        for i in range(config.num_layers):
            window = config.window_size_for_layer(i)
            with ctx.scope(f"layers.{i}", unit=f"layers.{i}"):
                layers.append(config.layer.build(d, config.hidden_size, window_size=window, policy=policy,
                                                 init_std=config.init_std))
        self.layers = torch.nn.ModuleList(layers)
        with ctx.scope("norm", unit="head"):
            self.norm = config.norm.build(d)
        with ctx.scope("lm_head", unit="head"):
            tied = self.embedding.weight if config.tie_embeddings else None
            self.lm_head = config.lm_head.build(d, config.vocab_size, tied_weight=tied, init_std=config.init_std)
        if isinstance(policy, NamedCheckpointPolicy):
            policy.resolve_names(self.get_region_names())
        self._anchor: Optional[torch.Tensor] = None
        self.ce_chunk_rows = config.ce_chunk_rows

    # ------------------------------------------------------------------ helpers
    def get_region_names(self) -> List[str]:
        names = []
        for i in range(len(self.layers)):
            names += [f"layers.{i}", f"layers.{i}.attention", f"layers.{i}.mlp"]
        return names

    def get_buffer_cache(self, seq_len: int, device: Optional[torch.device] = None) -> BufferCache:
        """Precompute the RoPE tables for ``seq_len`` (``model.py:138-144``)."""
        cache = BufferCache()
        device = device if device is not None else self.store.device
        for layer in self.layers:
            rope = layer.attention.rope
            if rope is not None:
                rope.get_tables(seq_len, device, cache)
        return cache

    def num_params(self) -> int:
        return self.store.num_parameters()

    def num_flops_per_token(self, seq_len: int) -> int:
        """Training FLOPs per token: 6 x matmul parameters (LM head included, embedding gather excluded) plus the
        causal attention term 6 * L * H * D * S."""
        cfg = self.config
        matmul_params = 0
        for name, h in self.param_handles():
            if len(h.meta.shape) == 2 and not name.startswith("embedding."):
                matmul_params += h.meta.shape[0] * h.meta.shape[1]
        if cfg.tie_embeddings:
            matmul_params += cfg.vocab_size * cfg.d_model
        att = cfg.layer.attention
        hd = att.head_dim or cfg.d_model // att.n_heads
        return 6 * matmul_params + 6 * cfg.num_layers * att.n_heads * hd * seq_len

    def _unit(self, name: str) -> FSDPUnit:
        return self.store.unit(name)

    # ------------------------------------------------------------------ forward
    def _trunk(self, ids: torch.Tensor, cache: Optional[BufferCache]) -> Tuple[torch.Tensor, int]:
        """ids [B, S] -> final-normed hidden states [tokens_local, d]."""
        B, S = ids.shape
        tp = self.mesh.tp
        flat = ids.reshape(-1)
        if tp.size > 1:
            flat = flat.chunk(tp.size)[tp.rank]
        emb_unit = self._unit("embedding")
        emb_unit.start_gather()
        self.store.prefetch(emb_unit.index + 1)
        if self._anchor is None or self._anchor.device != ids.device:
            self._anchor = torch.zeros(1, device=ids.device, requires_grad=True)
        anchor = self._anchor if torch.is_grad_enabled() else None
        x = self.embedding(flat, anchor)
        x, _ = _exit(x, None, emb_unit)
        delta = None
        for i, layer in enumerate(self.layers):
            unit = self._unit(f"layers.{i}")
            x, delta = _enter(x, delta, unit)
            x, delta = layer(x, delta, B, cache)
            x, delta = _exit(x, delta, unit)
        head_unit = self._unit("head")
        x, delta = _enter(x, delta, head_unit)
        if delta is not None:
            _, x = self.norm(delta, residual=x, mode="pre")
        else:
            x = self.norm(x)
        return x, B

    def forward(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None, cache: Optional[BufferCache] = None,
                ignore_index: int = -100, z_loss_multiplier: float = 0.0):
        """
        With ``labels``: returns ``(loss, z_loss)``, the mean cross entropy over this rank's tokens computed by the
        fused LM-head + loss (logits are not materialised).  Without: returns fp32 logits ``[B, S(/tp), V]``.
        """
        x, B = self._trunk(ids, cache)
        head_unit = self._unit("head")
        if self.config.tie_embeddings:
            self._unit("embedding").gathered()
        if labels is None:
            logits = self.lm_head(x)
            return logits.view(B, -1, logits.shape[-1]) if self.mesh.tp.size == 1 else logits
        lab = labels.reshape(-1)
        tp = self.mesh.tp
        if tp.size > 1:
            lab = lab.chunk(tp.size)[tp.rank]
        loss, zl = self.lm_head.loss(x, lab, ignore_index=ignore_index, z_loss_multiplier=z_loss_multiplier,
                                     chunk_rows=self.ce_chunk_rows)
        if self.store.reshard_after_forward and self.store.mesh.shard.size > 1 and not torch.is_grad_enabled():
            head_unit.release()
        return loss, zl


@dataclass
class TransformerConfig(Registrable):
    vocab_size: int = 50304
    d_model: int = 1024
    hidden_size: int = 2816
    num_layers: int = 16
    layer: TransformerLayerConfig = field(default_factory=DefaultTransformerLayerConfig)
    norm: NormalizerConfig = field(default_factory=RMSNormConfig)
    lm_head: LMHeadConfig = field(default_factory=LMHeadConfig)
    scan_layers: bool = False
    """Accepted for compatibility: there is no trace/compile step whose time a scan would save."""
    layer_ac_policy: Optional[ActivationCheckpointingPolicy] = None
    tie_embeddings: bool = False
    scale_embeddings: bool = False
    """Multiply embedding outputs by sqrt(d_model) (Gemma)."""
    sliding_window: Optional[int] = None
    sliding_window_pattern: int = 1
    """With ``sliding_window`` set: layer i uses the window unless ``(i + 1) % pattern == 0`` (pattern 1: every layer
    windowed; pattern 2: windowed and global layers alternate, starting with a windowed one)."""
    init_std: float = 0.02
    ce_chunk_rows: int = 2048

    def window_size_for_layer(self, i: int) -> Optional[int]:
        if self.sliding_window is None:
            return self.layer.attention.window_size
        if self.sliding_window_pattern > 1 and (i + 1) % self.sliding_window_pattern == 0:
            return None
        return self.sliding_window

    def build(
        self,
        seed: int = 0,
        mesh: Optional[DeviceMesh] = None,
        *,
        mesh_resource: Optional[MeshResource] = None,
        param_dtype: torch.dtype = torch.float32,
        compute_dtype: Optional[torch.dtype] = None,
        device: Optional[torch.device] = None,
        reshard_after_forward: bool = True,
        comm_backend: Optional[str] = None,
        init: bool = True,
        **overrides,
    ) -> Transformer:
        cfg = dataclasses.replace(self, **overrides) if overrides else self
        if mesh is None:
            mesh = get_mesh()
        if mesh is None:
            resource = mesh_resource or MeshResource.FSDP(dist_utils.get_world_size())
            mesh = resource.build(device=device)
        device = device if device is not None else mesh.device
        if compute_dtype is None:
            compute_dtype = torch.bfloat16 if torch.device(device).type == "cuda" else param_dtype
        store = ParamStore(mesh, param_dtype=param_dtype, compute_dtype=compute_dtype, device=torch.device(device),
                           reshard_after_forward=reshard_after_forward, comm_backend=comm_backend)
        with BuildContext(store):
            model = Transformer(cfg)
        store.finalize(seed=seed, init=init)
        # With the peer-memory backend the embedding rows are read from the GPU that owns them, so the (large)
        # embedding unit is only gathered when something else needs the full matrix (a tied LM head).
        store.unit("embedding").lazy = store.symm_ag is not None
        return model


@TransformerConfig.register("default", default=True)
@dataclass
class DefaultTransformerConfig(TransformerConfig):
    pass

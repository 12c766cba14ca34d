"""
Transformer layers (``olmax/nn/transformer/layer.py:1-350``): pre-norm (``default``), OLMo2 post-norm
(``reordered_norm``) and Gemma pre+post norm (``gemma``).  Activations are ``[tokens, d_model]``; residual additions
are fused into the RMSNorm kernels, so a layer issues no stand-alone elementwise add.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

from ..activation_checkpointing import ActivationCheckpointingPolicy, NoPolicy
from ..nn.attention import MultiheadSelfAttentionConfig
from ..nn.mlp import GatedMLP
from ..nn.module import Module, current_build_context
from ..nn.normalization import NormalizerConfig, RMSNormConfig
from ..nn.rope import BufferCache
from ..utils.dataclass_codec import Registrable

__all__ = [
    "TransformerLayer",
    "ReorderedNormTransformerLayer",
    "GemmaTransformerLayer",
    "TransformerLayerConfig",
    "DefaultTransformerLayerConfig",
    "ReorderedNormTransformerLayerConfig",
    "GemmaTransformerLayerConfig",
]


class _LayerBase(Module):
    activation = "silu"

    def __init__(self, cfg: "TransformerLayerConfig", d_model: int, hidden_size: int, window_size: Optional[int],
                 policy: ActivationCheckpointingPolicy, init_std: float):
        super().__init__()
        ctx = current_build_context()
        self.policy = policy
        with ctx.scope("attention"):
            self.attention = cfg.attention.build(d_model, window_size=window_size, init_std=init_std)
        with ctx.scope("mlp"):
            self.mlp = GatedMLP(d_model, hidden_size, bias=cfg.bias, activation=self.activation, init_std=init_std)
        self._layer_fn = policy.wrap(self._forward_impl, self.checkpoint_name)
        self._whole_layer = policy.should_recompute(self.checkpoint_name)
        # sub-block regions (`layers.i.attention`, `layers.i.mlp`): recomputed on their own unless the whole layer
        # already is (a nested checkpoint would run the sub-block's forward a third time)
        self._attn_fn, self._mlp_fn = self._attention_block, self._mlp_block
        if not self._whole_layer:
            # the attention block rebuilds q / k / v inside its own autograd node (neither the attention forward nor the
            # output projection runs again); only under context parallelism is it wrapped in a checkpoint
            if self.attention.recomputes_itself:
                self.attention.recompute = policy.should_recompute(f"{self.checkpoint_name}.attention")
            else:
                self._attn_fn = policy.wrap(self._attention_block, f"{self.checkpoint_name}.attention")
            # the MLP block recomputes inside its own autograd node (only its gate/up GEMM runs again) instead of being
            # wrapped in a checkpoint, which would also repeat the down projection
            self.mlp.recompute = policy.should_recompute(f"{self.checkpoint_name}.mlp")

    def _norm(self, name: str, cfg: "TransformerLayerConfig", size: int):
        with current_build_context().scope(name):
            return cfg.norm.build(size)

    def _attention_block(self, x, batch_size, cache):
        return self.attention(x, batch_size, cache)

    def _mlp_block(self, x):
        return self.mlp(x)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch_size: int,
                cache: Optional[BufferCache] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """
        The layer input is ``x + delta`` (``delta`` is a residual branch the previous layer left un-added so that the
        addition can be fused into this layer's first norm; None when there is nothing pending).  Returns the same
        kind of pair.
        """
        if self._whole_layer and torch.is_grad_enabled():
            if delta is None:
                return self._layer_fn(x, None, batch_size, cache)
            return self._layer_fn(x, delta, batch_size, cache)
        return self._forward_impl(x, delta, batch_size, cache)


class TransformerLayer(_LayerBase):
    """Pre-norm: ``h = x + attn(norm(x)); out = h + mlp(norm(h))`` (``layer.py:80-94``)."""

    def __init__(self, cfg, d_model, hidden_size, window_size, policy, init_std):
        super().__init__(cfg, d_model, hidden_size, window_size, policy, init_std)
        self.attention_norm = self._norm("attention_norm", cfg, d_model)
        self.mlp_norm = self._norm("mlp_norm", cfg, d_model)

    def _forward_impl(self, x, delta, batch_size, cache):
        if delta is not None:
            x, n = self.attention_norm(delta, residual=x, mode="pre")
        else:
            n = self.attention_norm(x)
        a = self._attn_fn(n, batch_size, cache)
        h, n2 = self.mlp_norm(a, residual=x, mode="pre")
        m = self._mlp_fn(n2)
        return h, m


class ReorderedNormTransformerLayer(_LayerBase):
    """OLMo2: ``h = x + norm(attn(x)); out = h + norm(mlp(h))`` (``layer.py:102-116``)."""

    def __init__(self, cfg, d_model, hidden_size, window_size, policy, init_std):
        super().__init__(cfg, d_model, hidden_size, window_size, policy, init_std)
        self.attention_norm = self._norm("attention_norm", cfg, d_model)
        self.mlp_norm = self._norm("mlp_norm", cfg, d_model)

    def _forward_impl(self, x, delta, batch_size, cache):
        assert delta is None
        a = self._attn_fn(x, batch_size, cache)
        h = self.attention_norm(a, residual=x, mode="post")
        m = self._mlp_fn(h)
        out = self.mlp_norm(m, residual=h, mode="post")
        return out, None


class GemmaTransformerLayer(_LayerBase):
    """Gemma: ``h = x + post(attn(pre(x))); out = h + post(mlp(pre(h)))`` with GeGLU (``layer.py:119-185``)."""

    activation = "gelu_tanh"

    def __init__(self, cfg, d_model, hidden_size, window_size, policy, init_std):
        super().__init__(cfg, d_model, hidden_size, window_size, policy, init_std)
        self.attention_input_norm = self._norm("attention_input_norm", cfg, d_model)
        self.attention_norm = self._norm("attention_norm", cfg, d_model)
        self.mlp_input_norm = self._norm("mlp_input_norm", cfg, d_model)
        self.mlp_norm = self._norm("mlp_norm", cfg, d_model)

    def _forward_impl(self, x, delta, batch_size, cache):
        assert delta is None
        a = self._attn_fn(self.attention_input_norm(x), batch_size, cache)
        h = self.attention_norm(a, residual=x, mode="post")
        m = self._mlp_fn(self.mlp_input_norm(h))
        out = self.mlp_norm(m, residual=h, mode="post")
        return out, None


@dataclass
class TransformerLayerConfig(Registrable):
    attention: MultiheadSelfAttentionConfig = field(default_factory=MultiheadSelfAttentionConfig)
    norm: NormalizerConfig = field(default_factory=RMSNormConfig)
    bias: bool = False

    layer_class = TransformerLayer

    def build(self, d_model: int, hidden_size: int, window_size: Optional[int] = "inherit",
              policy: Optional[ActivationCheckpointingPolicy] = None, init_std: float = 0.02) -> _LayerBase:
        return self.layer_class(self, d_model, hidden_size, window_size, policy or NoPolicy(), init_std)


@TransformerLayerConfig.register("default", default=True)
@dataclass
class DefaultTransformerLayerConfig(TransformerLayerConfig):
    layer_class = TransformerLayer


@TransformerLayerConfig.register("reordered_norm")
@dataclass
class ReorderedNormTransformerLayerConfig(TransformerLayerConfig):
    layer_class = ReorderedNormTransformerLayer


@TransformerLayerConfig.register("gemma")
@dataclass
class GemmaTransformerLayerConfig(TransformerLayerConfig):
    layer_class = GemmaTransformerLayer

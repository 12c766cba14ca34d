"""
Model recipes (``olmax/nn/transformer/recipes.py:1-360``): the reference's eight recipes with their per-device
micro-batch sizes, plus the benchmark variants of four of them (names ending in ``_bench``) that add what the
benchmark configurations ask for and the reference recipes lack: vocabulary padded to a multiple of the shard count,
RoPE theta 500000, OLMo2 QK-norm over the full projections, Gemma2's alternating sliding-window / global attention,
logit soft-caps, tied and scaled embeddings; and a tiny CPU recipe used by the multi-process tests.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Optional

from ..activation_checkpointing import NothingSaveable
from ..env import EnvConfig
from ..nn.attention import MultiheadSelfAttentionConfig
from ..nn.lm_head import LMHeadConfig
from ..nn.normalization import RMSNormConfig
from ..nn.rope import RotaryPositionalEmbeddingConfig
from ..types import DeviceType, StrEnum
from .layer import (
    DefaultTransformerLayerConfig,
    GemmaTransformerLayerConfig,
    ReorderedNormTransformerLayerConfig,
)
from .model import DefaultTransformerConfig, TransformerConfig

__all__ = ["TransformerRecipeType", "TransformerRecipe"]


class TransformerRecipeType(StrEnum):
    llama_like_271M = "llama_like_271M"
    llama_like_7B = "llama_like_7B"
    llama3_8B = "llama3_8B"
    llama3_70B = "llama3_70B"
    olmo2_7B = "olmo2_7B"
    olmo2_32B = "olmo2_32B"
    gemma2_like_27B = "gemma2_like_27B"
    gemma3_like_27B = "gemma3_like_27B"
    # benchmark variants and the CPU test model
    llama_like_7B_bench = "llama_like_7B_bench"
    olmo2_7B_bench = "olmo2_7B_bench"
    olmo2_32B_bench = "olmo2_32B_bench"
    gemma2_like_27B_bench = "gemma2_like_27B_bench"
    tiny_llama = "tiny_llama"

    def build_recipe(self, env_defaults: Optional[EnvConfig] = None,
                     device_type: DeviceType = DeviceType.NVIDIA_B200) -> "TransformerRecipe":
        env = env_defaults if env_defaults is not None else EnvConfig()
        return getattr(TransformerRecipe, self.value)(env_defaults=env, device_type=device_type)


def _mbz(device_type: DeviceType, table: dict, recipe: str) -> int:
    if device_type not in table:
        raise NotImplementedError(f"recipe {recipe} has no default micro-batch size for device type {device_type}")
    return table[device_type]


_K = 1024
_NORM = RMSNormConfig(eps=1e-5, use_bias=False)


def _decoder(vocab, d, hidden, layers, heads, kv_heads, theta, layer_cls, qk_norm=False, head_qk_norm=True, **kw):
    attn = MultiheadSelfAttentionConfig(
        n_heads=heads,
        n_kv_heads=kv_heads if kv_heads != heads else None,
        head_dim=128,
        rope=RotaryPositionalEmbeddingConfig(theta=theta),
        bias=False,
        qk_norm=RMSNormConfig() if qk_norm else None,
        use_head_qk_norm=head_qk_norm if qk_norm else False,
        logit_softcap=kw.pop("attn_softcap", None),
    )
    lm_head = LMHeadConfig(bias=False, logit_softcap=kw.pop("final_softcap", None))
    return DefaultTransformerConfig(
        vocab_size=vocab, d_model=d, hidden_size=hidden, num_layers=layers,
        layer=layer_cls(attention=attn, norm=RMSNormConfig(), bias=False),
        norm=RMSNormConfig(), lm_head=lm_head, **kw,
    )


@dataclass
class TransformerRecipe:
    model: TransformerConfig
    sequence_length: int
    local_microbatch_size: int
    """Tokens per device per micro-batch."""
    env: EnvConfig = field(default_factory=EnvConfig)

    # ------------------------------------------------------------------ the reference's recipes
    @classmethod
    def llama_like_271M(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_A100_40GB: 16 * _K, DeviceType.NVIDIA_H100: 32 * _K,
                                 DeviceType.NVIDIA_B200: 64 * _K}, "llama_like_271M")
        return cls(_decoder(50304, 1024, 2816, 16, 8, 8, 10_000.0, DefaultTransformerLayerConfig), 1024, mbz, env_defaults)

    @classmethod
    def llama_like_7B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_H100: 2 * 4096, DeviceType.NVIDIA_B200: 4 * 4096}, "llama_like_7B")
        env = dataclasses.replace(env_defaults)
        env.xla.gpu_all_gather_combine_threshold_mib = 1024
        env.xla.gpu_all_reduce_combine_threshold_mib = 1024
        return cls(_decoder(50304, 4096, 11008, 32, 32, 32, 10_000.0, DefaultTransformerLayerConfig), 4096, mbz, env)

    @classmethod
    def llama3_8B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_H100: 8192, DeviceType.NVIDIA_B200: 2 * 8192}, "llama3_8B")
        return cls(_decoder(128256, 4096, 14336, 32, 32, 8, 500_000.0, DefaultTransformerLayerConfig), 8192, mbz, env_defaults)

    @classmethod
    def llama3_70B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_H100: 8192, DeviceType.NVIDIA_B200: 8192}, "llama3_70B")
        model = _decoder(128256, 8192, 28672, 80, 64, 8, 500_000.0, DefaultTransformerLayerConfig,
                         scan_layers=True, layer_ac_policy=NothingSaveable(prevent_cse=False))
        return cls(model, 8192, mbz, env_defaults)

    @classmethod
    def olmo2_7B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_H100: 2 * 4096, DeviceType.NVIDIA_B200: 4 * 4096}, "olmo2_7B")
        return cls(_decoder(100278, 4096, 11008, 32, 32, 32, 10_000.0, ReorderedNormTransformerLayerConfig,
                            qk_norm=True, head_qk_norm=True), 4096, mbz, env_defaults)

    @classmethod
    def olmo2_32B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_H100: 4 * 4096, DeviceType.NVIDIA_B200: 4 * 4096}, "olmo2_32B")
        model = _decoder(100278, 5120, 27648, 64, 40, 8, 10_000.0, ReorderedNormTransformerLayerConfig, qk_norm=True,
                         head_qk_norm=True, scan_layers=True, layer_ac_policy=NothingSaveable(prevent_cse=False))
        return cls(model, 4096, mbz, env_defaults)

    @classmethod
    def gemma2_like_27B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_B200: 2 * 4096}, "gemma2_like_27B")
        return cls(_decoder(256000, 4608, 36864, 46, 32, 16, 10_000.0, GemmaTransformerLayerConfig), 4096, mbz, env_defaults)

    @classmethod
    def gemma3_like_27B(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        mbz = _mbz(device_type, {DeviceType.NVIDIA_B200: 2 * 4096}, "gemma3_like_27B")
        return cls(_decoder(256000, 5376, 21504, 62, 32, 16, 10_000.0, GemmaTransformerLayerConfig, qk_norm=True,
                            head_qk_norm=True), 4096, mbz, env_defaults)

    # ------------------------------------------------------------------ benchmark variants
    @classmethod
    def llama_like_7B_bench(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        """Llama-like 7B as benchmarked: vocabulary 100352, RoPE theta 500000, 2 x 4096 tokens per GPU."""
        return cls(_decoder(100352, 4096, 11008, 32, 32, 32, 500_000.0, DefaultTransformerLayerConfig), 4096, 2 * 4096,
                   env_defaults)

    @classmethod
    def olmo2_7B_bench(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        """OLMo2 7B as benchmarked: vocabulary 100352, theta 500000, QK-norm over the full q / k projections."""
        return cls(_decoder(100352, 4096, 11008, 32, 32, 32, 500_000.0, ReorderedNormTransformerLayerConfig,
                            qk_norm=True, head_qk_norm=False), 4096, 2 * 4096, env_defaults)

    @classmethod
    def olmo2_32B_bench(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        """OLMo2 32B as benchmarked: vocabulary 100352, theta 500000, full per-block recomputation, 4 x 4096 tokens."""
        model = _decoder(100352, 5120, 27648, 64, 40, 8, 500_000.0, ReorderedNormTransformerLayerConfig, qk_norm=True,
                         head_qk_norm=True, layer_ac_policy=NothingSaveable(prevent_cse=False))
        return cls(model, 4096, 4 * 4096, env_defaults)

    @classmethod
    def gemma2_like_27B_bench(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        """Gemma2-like 27B as benchmarked: sliding window 4096 alternating with global attention, attention soft-cap
        50, final-logit soft-cap 30, tied embeddings scaled by sqrt(d_model)."""
        model = _decoder(256000, 4608, 36864, 46, 32, 16, 10_000.0, GemmaTransformerLayerConfig, attn_softcap=50.0,
                         final_softcap=30.0, tie_embeddings=True, scale_embeddings=True, sliding_window=4096,
                         sliding_window_pattern=2)
        return cls(model, 4096, 2 * 4096, env_defaults)

    @classmethod
    def tiny_llama(cls, env_defaults: EnvConfig, device_type: DeviceType) -> "TransformerRecipe":
        """2 layers, d_model 256, 4 heads x 64, SwiGLU 688, RMSNorm eps 1e-6, theta 10000, vocabulary 1024, seq 256."""
        attn = MultiheadSelfAttentionConfig(n_heads=4, head_dim=64, rope=RotaryPositionalEmbeddingConfig(theta=10_000.0))
        norm = RMSNormConfig(eps=1e-6)
        model = DefaultTransformerConfig(vocab_size=1024, d_model=256, hidden_size=688, num_layers=2,
                                         layer=DefaultTransformerLayerConfig(attention=attn, norm=norm), norm=norm,
                                         lm_head=LMHeadConfig())
        return cls(model, 256, 256, env_defaults)

from . import functional, init
from .attention import AttentionImplementation, AttentionKernel, MultiheadSelfAttention, MultiheadSelfAttentionConfig
from .embedding import Embedding
from .linear import Linear
from .lm_head import LMHead, LMHeadConfig
from .mlp import GatedMLP
from .module import BuildContext, Module
from .normalization import LayerNorm, LayerNormConfig, Normalizer, NormalizerConfig, RMSNorm, RMSNormConfig
from .rope import BufferCache, RotaryPositionalEmbedding, RotaryPositionalEmbeddingConfig

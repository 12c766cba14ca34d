from .layer import (
    DefaultTransformerLayerConfig,
    GemmaTransformerLayerConfig,
    ReorderedNormTransformerLayer,
    ReorderedNormTransformerLayerConfig,
    GemmaTransformerLayer,
    TransformerLayer,
    TransformerLayerConfig,
)
from .model import DefaultTransformerConfig, Transformer, TransformerConfig
from .recipes import TransformerRecipe, TransformerRecipeType

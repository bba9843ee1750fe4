"""Model families: the reference's modules (Linear ... GPT), the MLP classifier and the Mars
demo model, plus the 350M / 1.3B GPT presets used by the multi-GPU configurations."""
from .gpt import GPT, PRESETS, build_preset
from .layers import (Embedding, FeedForward, LayerNorm, Linear, Module, MultiHeadAttention, SelfAttention,
                     TransformerBlock)
from .mars import Mars
from .mlp import MLP

__all__ = ["GPT", "PRESETS", "build_preset", "Embedding", "FeedForward", "LayerNorm", "Linear", "Module",
           "MultiHeadAttention", "SelfAttention", "TransformerBlock", "Mars", "MLP"]

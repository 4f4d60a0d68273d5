"""Model families: the Llama-3-shaped flagship and the README-style SimpleTransformer."""
from .llama import FlatBuffers, LlamaConfig, LlamaModel, RematPolicy
from .simple_transformer import SimpleTransformer

__all__ = ["LlamaConfig", "LlamaModel", "RematPolicy", "FlatBuffers", "SimpleTransformer"]

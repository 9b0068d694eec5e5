"""Model definitions used by the benchmarks and smoke tests."""

from .gpt2 import GPT2, GPT2Config
from .llama import Llama, LlamaConfig
from .mlp import SyntheticMLP

__all__ = ["GPT2", "GPT2Config", "Llama", "LlamaConfig", "SyntheticMLP"]

"""Models: the Llama family on this package's kernels, a GPT-style decoder, and a small zoo."""

from .llama import LLAMA_CONFIGS, LlamaConfig, build_llama, build_llama_stages, llama_loss_fn
from .gpt import GPT, GPTConfig, gpt_stages

__all__ = ["LLAMA_CONFIGS", "LlamaConfig", "build_llama", "build_llama_stages", "llama_loss_fn", "GPT", "GPTConfig", "gpt_stages"]

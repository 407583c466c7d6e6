from . import debuvik, dezolorn, llama, sorizen  # registers Debuvik, Dezolorn, LlamaForCausalLM and Sorizen

__all__ = ["debuvik", "dezolorn", "llama", "sorizen"]

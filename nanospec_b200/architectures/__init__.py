from . import debuvik, dezolorn, fubolix, llama, sorizen  # registers Debuvik, Dezolorn, Fubolix, LlamaForCausalLM and Sorizen

__all__ = ["debuvik", "dezolorn", "fubolix", "llama", "sorizen"]

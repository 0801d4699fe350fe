"""Model builders for the benchmark configurations: the 784-256-128-10 MLP, the small CNN and
the decoder-only causal language model (tiny and ~1.3 B presets)."""
from .mlp import MLP  # noqa: F401
from .cnn import SmallCNN  # noqa: F401
from .causal_lm import CausalLM, CausalLMConfig, TINY_LM, LM_1P3B  # noqa: F401

r"""Model families the reference ships as examples: a Megatron-shaped GPT (for ``fmoefy``)
and Transformer-XL with MoE feed-forward blocks."""
from .gpt import GPTConfig, GPTModel  # noqa: F401
from .transformer_xl import MemTransformerLM  # noqa: F401

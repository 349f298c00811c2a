from .rotary import RotaryEmbedding, get_rope

__all__ = ("RotaryEmbedding", "get_rope")

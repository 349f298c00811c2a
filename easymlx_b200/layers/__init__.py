from .rotary import LongRopeEmbedding, RotaryEmbedding, get_rope

__all__ = ("LongRopeEmbedding", "RotaryEmbedding", "get_rope")

from ..utils.registry import Registry

ATTENTION = Registry("attention")
FFN = Registry("ffn")
NORM = Registry("norm")
ROPE = Registry("rope")
EMBEDDING = Registry("embedding")

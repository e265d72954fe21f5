from .core import (Embedding, GQAPlain, GQAQKNorm, Linear, RMSNorm, RoPE, RoPEYarn, SwiGLU, UntiedEmbedding)

"""`repop.nn.embedding.Embedding` (reference: model/modules/embedding_repop.py:28,36)."""
import torch.nn as nn


class Embedding(nn.Embedding):
    pass

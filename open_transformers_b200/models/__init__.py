from .fused_loss import cross_entropy, fused_ce_z_loss, streaming_head_loss
from .init import init_weights
from .llama3 import Llama3, ModelOutput, TransformerBlock, build_model
from .registry import ATTENTION, EMBEDDING, FFN, NORM, ROPE

__all__ = ["Llama3", "ModelOutput", "TransformerBlock", "build_model", "init_weights", "fused_ce_z_loss",
           "cross_entropy", "streaming_head_loss", "ATTENTION", "FFN", "NORM", "ROPE", "EMBEDDING"]

from .attention import BaseAttention, GQAttention
from .decoder import Decoder, TransformerBlock
from .embedding import Embedding
from .feed_forward import FeedForward, compute_ffn_hidden_dim
from .linear import Linear
from .rmsnorm import RMSNorm
from .rope import RoPE, apply_rotary_emb

__all__ = [
    "BaseAttention",
    "GQAttention",
    "Decoder",
    "TransformerBlock",
    "Embedding",
    "FeedForward",
    "compute_ffn_hidden_dim",
    "Linear",
    "RMSNorm",
    "RoPE",
    "apply_rotary_emb",
]

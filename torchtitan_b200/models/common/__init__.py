from .attention import (
    BaseAttention,
    GQAttention,
    create_attention_mask,
    create_varlen_metadata_for_document,
    get_causal_mask_mod,
    get_document_mask_mod,
    get_fixed_block_mask_mod,
    get_sliding_window_mask_mod,
)
from .decoder import Decoder, TransformerBlock
from .embedding import Embedding
from .feed_forward import FeedForward, compute_ffn_hidden_dim
from .linear import Linear
from .rmsnorm import RMSNorm
from .moe import MoE
from .rope import RoPE, apply_rotary_emb, apply_rotary_emb_complex, apply_rotary_emb_cos_sin, apply_rotary_emb_single_complex

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
    "apply_rotary_emb_complex",
    "apply_rotary_emb_cos_sin",
    "apply_rotary_emb_single_complex",
    "MoE",
    "create_attention_mask",
    "create_varlen_metadata_for_document",
    "get_causal_mask_mod",
    "get_document_mask_mod",
    "get_fixed_block_mask_mod",
    "get_sliding_window_mask_mod",
]

"""Grouped-query attention block and the mask descriptions it understands.

Parity: torchtitan/models/common/attention.py:378-570 (config fields, projection names
``wq/wk/wv/wo``, optional per-head QK RMSNorm before RoPE, ``scale`` only when ``head_dim`` is
explicit, ``attn_backend`` in {sdpa, flex, varlen} and ``attn_mask_type`` in {causal,
block_causal}); mask builders :215-375 (causal, document, fixed block, sliding window).

All three backends end in the same flash-attention kernel here; what differs is the mask
description handed to it (:class:`AttentionMasks`): nothing for plain causal, per-token
document ids for block-causal ("flex") or the cumulative sequence lengths form ("varlen"),
plus an optional sliding window / fixed block size. Tensors stay ``[B, S, H, Dh]``; the kernel
reads that layout through strided TMA descriptors, so no transposes are materialised.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module

from .linear import Linear, project_together
from .rmsnorm import RMSNorm
from .rope import apply_rotary_emb


@dataclass
class AttentionMasks:
    """Sparse-mask description consumed by ``ops.attention`` (all optional).

    doc_ids     int32 [B, S]: tokens attend only within equal ids (document masking)
    cu_seqlens  int32 [n_docs + 1]: the same information in packed form (varlen backend)
    window      sliding window length
    block       fixed block size: attention never crosses multiples of ``block``
    """

    doc_ids: torch.Tensor | None = None
    cu_seqlens: torch.Tensor | None = None
    max_seqlen: int | None = None
    window: int | None = None
    block: int | None = None


AttentionMasksType = AttentionMasks | dict[str, AttentionMasks]


def document_ids(tokens: torch.Tensor, eos_id: int) -> torch.Tensor:
    """Document index of every token: a document ends *with* its EOS token."""
    is_eos = tokens == eos_id
    ends = torch.cumsum(is_eos.to(torch.int32), dim=1)
    return (ends - is_eos.to(torch.int32)).to(torch.int32)


def fixed_block_ids(batch: int, seqlen: int, block: int, device=None) -> torch.Tensor:
    return (torch.arange(seqlen, device=device, dtype=torch.int32) // block).expand(batch, seqlen)


def create_varlen_metadata_for_document(tokens: torch.Tensor, eos_id: int) -> AttentionMasks:
    """Packed description: boundaries after each EOS and at each row end, over the flattened batch."""
    B, S = tokens.shape
    ids = document_ids(tokens, eos_id) + (torch.arange(B, device=tokens.device, dtype=torch.int32) * (S + 1)).view(B, 1)
    flat = ids.flatten()
    change = torch.ones_like(flat, dtype=torch.bool)
    change[1:] = flat[1:] != flat[:-1]
    starts = torch.nonzero(change).flatten().to(torch.int32)
    cu = torch.cat((starts, torch.tensor([B * S], dtype=torch.int32, device=tokens.device)))
    max_len = int((cu[1:] - cu[:-1]).max())
    dense = torch.cumsum(change.to(torch.int32), 0).view(B, S) - 1
    return AttentionMasks(doc_ids=dense.to(torch.int32), cu_seqlens=cu, max_seqlen=max_len)


class InnerAttention(Module):
    """The softmax(QK^T)V core as a module of its own so that context parallel can wrap it.

    Parity: the ``inner_attention`` wrapper modules of torchtitan/models/common/attention.py:48-212.
    """

    def __init__(self):
        super().__init__()
        self.ring = None  # set by parallel.cp.apply_cp_to_attention_module

    def forward(self, q, k, v, *, masks: AttentionMasks | None = None, scale=None, sinks=None, window=None):
        doc_ids = None
        if masks is not None:
            doc_ids = masks.doc_ids
            window = masks.window if masks.window is not None else window
            if masks.block is not None:
                if self.ring is not None:
                    raise NotImplementedError("fixed-block attention masks are built from local positions; "
                                              "context parallel serves document, window and sink masks")
                blocks = fixed_block_ids(q.shape[0], q.shape[1], masks.block, q.device)
                # both constraints: same document AND same fixed block <=> equal combined ids
                doc_ids = blocks if doc_ids is None else doc_ids * (q.shape[1] // masks.block + 1) + blocks
        if self.ring is not None:
            return self.ring(q, k, v, scale=scale, doc_ids=doc_ids, window=window, sinks=sinks)
        return ops.attention(q, k, v, causal=True, scale=scale, window=window, doc_ids=doc_ids, sinks=sinks)

    def init_weights(self, **kwargs) -> None:
        return None


class BaseAttention(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        n_heads: int
        attn_backend: str
        attn_mask_type: str

        def __post_init__(self):
            assert self.n_heads > 0, "n_heads must be > 0"
            assert self.attn_backend in ("flex", "varlen", "sdpa"), (
                f"attn_backend must be one of ['flex', 'varlen', 'sdpa'], got {self.attn_backend}"
            )
            assert self.attn_mask_type in ("causal", "block_causal"), (
                f"attn_mask_type must be one of ['causal', 'block_causal'], got {self.attn_mask_type}"
            )
            if self.attn_backend == "sdpa" and self.attn_mask_type == "block_causal":
                raise ValueError("attn_mask_type 'block_causal' is not supported with attn_backend 'sdpa'")


class GQAttention(BaseAttention):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseAttention.Config):
        n_heads: int
        q_norm: RMSNorm.Config | None = None
        k_norm: RMSNorm.Config | None = None
        n_kv_heads: int | None = None
        head_dim: int | None = None
        linear_bias: bool = False
        use_rope: bool = True
        attn_backend: str = "sdpa"
        attn_mask_type: str = "causal"
        rope_backend: str = "complex"

        def __post_init__(self):
            BaseAttention.Config.__post_init__(self)
            if (self.q_norm is None) != (self.k_norm is None):
                raise ValueError("q_norm and k_norm must be both None or both set")

    def __init__(self, config: Config, *, dim: int):
        super().__init__()
        self.n_heads = config.n_heads
        self.n_kv_heads = config.n_kv_heads or config.n_heads
        self.head_dim = config.head_dim if config.head_dim is not None else dim // config.n_heads
        self.enable_gqa = self.n_heads > self.n_kv_heads
        self.use_rope = config.use_rope
        self.rope_backend = config.rope_backend
        self.rope_layout = "interleaved" if config.rope_backend == "complex" else "half"
        self.attn_backend = config.attn_backend
        self.scaling = self.head_dim**-0.5 if config.head_dim is not None else None

        self.q_norm = self.k_norm = None
        if config.q_norm is not None:
            self.q_norm = config.q_norm.build(normalized_shape=self.head_dim)
            self.k_norm = config.k_norm.build(normalized_shape=self.head_dim)

        lin = Linear.Config(bias=config.linear_bias)
        self.wq = lin.build(in_features=dim, out_features=self.n_heads * self.head_dim)
        self.wk = lin.build(in_features=dim, out_features=self.n_kv_heads * self.head_dim)
        self.wv = lin.build(in_features=dim, out_features=self.n_kv_heads * self.head_dim)
        self.wo = lin.build(in_features=self.n_heads * self.head_dim, out_features=dim)
        self.inner_attention = InnerAttention()

    def forward(self, x, rope_cache, attention_masks: AttentionMasksType | None, positions=None, residual=None):
        """``residual``: the block's skip connection, added to the output projection (inside its GEMM where possible)."""
        bs, seqlen, _ = x.shape
        # asynchronous tensor parallel (parallel/tp.py): ``x`` is this rank's sequence shard, the projections gather it
        # inside the GEMM and ``wo`` reduce-scatters inside its GEMM
        fused_tp = self.__dict__.get("_fused_tp_call")
        if fused_tp is not None:
            q2, k2, v2 = fused_tp.project(self, x)
            seqlen = q2.shape[1]
            xq, xk, xv = (t.view(bs, seqlen, -1, self.head_dim) for t in (q2, k2, v2))
        else:
            # -1 for the head count: tensor parallel shards the projections by heads
            xq, xk, xv = (t.view(bs, seqlen, -1, self.head_dim) for t in project_together(x, self.wq, self.wk, self.wv))
        if self.q_norm is not None:
            xq, xk = self.q_norm(xq), self.k_norm(xk)
        if self.use_rope:
            xq, xk = apply_rotary_emb(xq, xk, rope_cache, positions, self.rope_layout)
        if isinstance(attention_masks, dict):
            attention_masks = attention_masks["rope" if self.use_rope else "nope"]
        if self.attn_backend == "sdpa":
            assert attention_masks is None
        else:
            assert isinstance(attention_masks, AttentionMasks), attention_masks
        out = self.inner_attention(xq, xk, xv, masks=attention_masks, scale=self.scaling)
        if fused_tp is not None:
            y = fused_tp.output(self, out.reshape(bs, seqlen, -1))
            return y if residual is None else residual + y
        out = out.reshape(bs, seqlen, -1)
        return self.wo(out) if residual is None else self.wo.add_to(residual, out)

    def init_weights(self, init_std: float = 0.02, **kwargs) -> None:
        for lin in (self.wq, self.wk, self.wv):
            lin.init_weights()
        self.wo.init_weights(init_std=init_std)
        if self.q_norm is not None:
            self.q_norm.init_weights()
            self.k_norm.init_weights()


# ------------------------------------------------------------------------------------------ mask functions
# The attention kernels of this framework take masks as per-row key ranges (``AttentionMasks``). Code written against the
# reference describes them as FlexAttention mask functions ``(batch, head, query index, key index) -> bool`` and builds
# block masks from them (torchtitan/models/common/attention.py:231-318); the same functions are offered here for models
# that call ``torch.nn.attention.flex_attention`` themselves.
def get_causal_mask_mod():
    def causal(b, h, q_idx, kv_idx):
        return q_idx >= kv_idx

    return causal


def get_document_mask_mod(batch: torch.Tensor, eos_id: int):
    """Tokens attend inside their own document; documents end with ``eos_id``."""
    docs = document_ids(batch, eos_id)

    def same_document(b, h, q_idx, kv_idx):
        return docs[b, q_idx] == docs[b, kv_idx]

    return same_document


def get_fixed_block_mask_mod(fixed_block_size: int):
    def same_block(b, h, q_idx, kv_idx):
        return (q_idx // fixed_block_size) == (kv_idx // fixed_block_size)

    return same_block


def get_sliding_window_mask_mod(window_size: int):
    if window_size < 1:
        raise ValueError(f"sliding window size must be at least 1, got {window_size}")

    def in_window(b, h, q_idx, kv_idx):
        return (kv_idx <= q_idx) & (q_idx - kv_idx < window_size)

    return in_window


def create_attention_mask(mask_mod, B, H, Q_LEN, KV_LEN, **kwargs):
    """FlexAttention block mask of a mask function (eager construction)."""
    from torch.nn.attention.flex_attention import create_block_mask

    return create_block_mask(mask_mod, B, H, Q_LEN, KV_LEN, **kwargs)

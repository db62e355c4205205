"""Decoder-only language model skeleton shared by the LM families.

Parity: torchtitan/models/common/decoder.py:37-208: ``tok_embeddings`` -> ``layers`` (a
``ModuleDict`` keyed by the layer index as a string, so pipeline stages can delete entries
without renumbering) -> ``norm`` -> ``output``; every top-level sub-module may be ``None``
after pipeline pruning and is then skipped; the RoPE table is a non-persistent buffer called
``freqs_cis``; the output projection is initialised with std ``dim**-0.5`` cut at 3 sigma.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.protocols.model import BaseModel
from torchtitan_b200.protocols.module import Module

from .attention import (
    AttentionMasks,
    AttentionMasksType,
    BaseAttention,
    create_varlen_metadata_for_document,
    document_ids,
)
from .embedding import Embedding
from .feed_forward import FeedForward
from .linear import Linear, with_residual
from .moe import MoE
from .rmsnorm import RMSNorm
from .rope import RoPE


class TransformerBlock(Module):
    """Pre-norm block: ``x + attn(norm(x))`` then ``h + ffn_or_moe(norm(h))``. Families
    subclass it for their own constructor / init rules."""

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        attention: BaseAttention.Config
        feed_forward: FeedForward.Config | None = None
        moe: MoE.Config | None = None
        attention_norm: RMSNorm.Config
        ffn_norm: RMSNorm.Config

    #: dense blocks hand their skip connections to the output projections, which add them in the GEMM epilogue
    fuse_residual = False

    def assemble(self, config, *, dim: int, layer_id: int, n_layers: int, attention=None, moe: bool = False,
                 depth_init: bool = True) -> None:
        """Sub-modules of the block: ``attention`` (built from ``attention`` when a family adjusts it per layer), either
        ``moe`` or ``feed_forward``, the two norms; output projections are initialised with ``0.02 / sqrt(2 d)`` where ``d``
        is the layer's depth (or the model's when ``depth_init`` is off)."""
        self.attention = (attention if attention is not None else config.attention).build(dim=dim)
        self.moe_enabled = moe
        part = config.moe if moe else config.feed_forward
        assert part is not None, "the block's configuration lacks its " + ("moe" if moe else "feed_forward") + " section"
        setattr(self, "moe" if moe else "feed_forward", part.build(dim=dim))
        self.attention_norm = config.attention_norm.build(normalized_shape=dim)
        self.ffn_norm = config.ffn_norm.build(normalized_shape=dim)
        self.weight_init_std = 0.02 / (2 * ((layer_id + 1) if depth_init else n_layers)) ** 0.5

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        if self.fuse_residual and not self.moe_enabled:
            h = with_residual(self.attention, x, self.attention_norm(x), freqs_cis, attention_masks, positions)
            return with_residual(self.feed_forward, h, self.ffn_norm(h))
        h = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
        return h + (self.moe if self.moe_enabled else self.feed_forward)(self.ffn_norm(h))

    def init_weights(self, **kwargs):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_weights(init_std=self.weight_init_std, buffer_device=kwargs.get("buffer_device"))
        else:
            self.feed_forward.init_weights(self.weight_init_std)


class Decoder(BaseModel):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseModel.Config):
        dim: int
        n_layers: int
        vocab_size: int
        output: Linear.Config
        tok_embeddings: Embedding.Config
        norm: RMSNorm.Config
        rope: RoPE.Config
        layer: TransformerBlock.Config

        def fit_to_job(self, trainer_config, *, context_parallel: bool = True) -> None:
            """What every decoder family adapts to a job: the rotary table covers the training sequence length, context
            parallel is refused for variable-length attention (or altogether), tensor parallel divides the head counts."""
            import dataclasses

            from torchtitan_b200.tools.logging import logger

            seq_len, par = trainer_config.training.seq_len, trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            backend = getattr(self.layer.attention, "attn_backend", None)
            if par.context_parallel_degree > 1 and (not context_parallel or backend == "varlen"):
                raise NotImplementedError(
                    "Context Parallel only supports SDPA and FlexAttention. "
                    f"Got attn_backend='{backend}'. Varlen attention is not supported with CP." if context_parallel else
                    f"Context Parallel is not supported for {type(self).__qualname__.split('.')[0]}.")
            tp, heads = par.tensor_parallel_degree, getattr(self.layer.attention, "n_heads", None)
            if tp > 1 and heads:
                kv = getattr(self.layer.attention, "n_kv_heads", None) or heads
                for name, n in (("n_heads", heads), ("n_kv_heads", kv)):
                    if n % tp != 0:
                        raise ValueError(f"tensor_parallel_degree ({tp}) must divide {name} ({n}).")

    def __init__(self, config: Config):
        super().__init__()
        self.config = config
        self.tok_embeddings = config.tok_embeddings.build(
            num_embeddings=config.vocab_size, embedding_dim=config.dim
        )
        self.rope = config.rope.build()
        self.register_buffer("freqs_cis", self.rope.cache, persistent=False)
        self.layers = nn.ModuleDict()
        for i in range(config.n_layers):
            self.layers[str(i)] = config.layer.build(layer_id=i, dim=config.dim, n_layers=config.n_layers)
        self.norm = config.norm.build(normalized_shape=config.dim)
        self.output = config.output.build(in_features=config.dim, out_features=config.vocab_size)

    def init_weights(self, **kwargs):
        buffer_device = kwargs.get("buffer_device") or self.freqs_cis.device
        rope = self.rope if self.rope is not None else self.config.rope.build()
        rope.init_weights(buffer_device=buffer_device)
        self.freqs_cis = rope.cache
        if self.tok_embeddings is not None:
            self.tok_embeddings.init_weights()
        for layer in self.layers.values():
            layer.init_weights(buffer_device=buffer_device)
        if self.norm is not None:
            self.norm.init_weights()
        if self.output is not None:
            std = self.config.dim**-0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def forward(self, tokens, attention_masks: AttentionMasksType | None = None, positions=None):
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, attention_masks, positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h

    # ---- masks --------------------------------------------------------------------
    @property
    def attn_config(self):
        return self.config.layer.attention

    def get_attention_masks(self, input_batch, tokenizer, extra_inputs=None) -> AttentionMasksType:
        cfg = self.attn_config
        if cfg.attn_backend == "flex":
            if cfg.attn_mask_type == "causal":
                return AttentionMasks()
            assert tokenizer.eos_id is not None
            return AttentionMasks(doc_ids=document_ids(input_batch, tokenizer.eos_id))
        if cfg.attn_backend == "varlen":
            if cfg.attn_mask_type != "block_causal":
                raise ValueError(
                    f"varlen attention is only supported with block_causal attention mask type, got {cfg.attn_mask_type}"
                )
            assert tokenizer.eos_id is not None
            return create_varlen_metadata_for_document(input_batch, tokenizer.eos_id)
        raise TypeError("Only varlen and flex attn masks are supported")

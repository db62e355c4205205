"""Llama 3 + SigLIP2-style encoder (torchtitan/experiments/vlm/model/{args,model,siglip2}.py)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.models.common.attention import AttentionMasks
from torchtitan_b200.models.llama3.model import Llama3Model
from torchtitan_b200.protocols.module import Module


@dataclass
class SpecialTokens:
    img_token: str
    img_id: int
    boi_token: str
    boi_id: int
    eoi_token: str
    eoi_id: int
    pad_token: str
    pad_id: int
    ignore_id: int = -100

    MAP = {"img": "<|image|>", "boi": "<|begin_of_image|>", "eoi": "<|end_of_image|>", "pad": "<|pad|>"}

    @classmethod
    def from_tokenizer(cls, tokenizer):
        out = {}
        for prefix, tok in cls.MAP.items():
            tid = tokenizer.token_to_id(tok)
            if tid is None:
                raise ValueError(f"tokenizer has no {tok} token")
            out[f"{prefix}_token"], out[f"{prefix}_id"] = tok, tid
        return cls(**out)


@dataclass
class Siglip2Config:
    dim: int = 768
    ffn_dim: int = 3072
    n_layers: int = 12
    n_heads: int = 12
    n_pos_embs: int = 16
    n_channels: int = 3
    patch_size: int = 16
    spatial_merge_size: int = 1
    layer_norm_eps: float = 1e-6
    attn_backend: str = "flex"
    attn_mask_type: str = "causal"
    """``causal`` / ``block_causal``: a patch attends to the patches before it in the image's row-major sequence, which is
    what the reference's encoder computes (torchtitan/experiments/vlm/model/siglip2.py:211-238 builds its mask from the
    causal mask function; its document variant splits at end-of-sequence ids, which a patch mask never holds);
    ``bidirectional``: every real patch of the image, as in the published SigLIP-2 encoder."""


def resize_positional_embeddings(pos_hwd: torch.Tensor, shapes_n2: torch.Tensor, max_length: int) -> torch.Tensor:
    """Bilinear (antialiased) resize of the learned H x W position grid to each image's patch grid, padded to ``max_length``."""
    _, _, D = pos_hwd.shape
    out = pos_hwd.new_zeros(shapes_n2.shape[0], max_length, D)
    grid = pos_hwd.permute(2, 0, 1).unsqueeze(0)
    cache: dict[tuple[int, int], torch.Tensor] = {}
    for i, (h, w) in enumerate(shapes_n2.tolist()):
        if h + w == 0:
            continue
        if (h, w) not in cache:
            r = F.interpolate(grid.float(), size=(h, w), mode="bilinear", align_corners=False, antialias=True)
            cache[(h, w)] = r[0].permute(1, 2, 0).reshape(h * w, D).to(pos_hwd.dtype)
        out[i, : h * w] = cache[(h, w)]
    return out


class VisionEmbeddings(Module):
    def __init__(self, a: Siglip2Config):
        super().__init__()
        self.patch_embedding = nn.Linear(a.n_channels * a.patch_size * a.patch_size, a.dim)
        self.position_embedding = nn.Embedding(a.n_pos_embs**2, a.dim)
        self.n_pos_embs = a.n_pos_embs

    def init_weights(self, **kwargs) -> None:
        nn.init.trunc_normal_(self.patch_embedding.weight, mean=0.0, std=0.02)
        nn.init.zeros_(self.patch_embedding.bias)
        nn.init.normal_(self.position_embedding.weight)

    def forward(self, pixels_nld, grid_hw):
        x = self.patch_embedding(pixels_nld)
        pos = self.position_embedding.weight.reshape(self.n_pos_embs, self.n_pos_embs, -1)
        shapes = torch.stack((grid_hw[:, :, 0].amax(1) + 1, grid_hw[:, :, 1].amax(1) + 1), dim=-1).long()
        return x + resize_positional_embeddings(pos, shapes, pixels_nld.shape[1])


class _EncoderAttention(Module):
    """Bidirectional multi-head attention over the patches of one image (parameter names as in the Hugging Face
    SigLIP-2 checkpoints and the reference's encoder: ``self_attn.{q,k,v,out}_proj``)."""

    def __init__(self, a: Siglip2Config):
        super().__init__()
        if a.attn_mask_type not in ("causal", "block_causal", "bidirectional"):
            raise ValueError(f"Unknown attention mask type: {a.attn_mask_type}")
        self.n_heads, self.causal = a.n_heads, a.attn_mask_type != "bidirectional"
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(a.dim, a.dim) for _ in range(4))

    def forward(self, h, key_mask):
        N, L, D = h.shape
        q, k, v = (p(h).view(N, L, self.n_heads, -1).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        if self.causal:      # padding patches come last, so real patches never see them
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            o = F.scaled_dot_product_attention(q, k, v, attn_mask=key_mask.view(N, 1, 1, L))
        return self.out_proj(o.transpose(1, 2).reshape(N, L, D))

    def init_weights(self, **kwargs) -> None:
        for m in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            nn.init.trunc_normal_(m.weight, mean=0.0, std=0.02)
            nn.init.zeros_(m.bias)


class _EncoderMLP(Module):
    def __init__(self, a: Siglip2Config):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(a.dim, a.ffn_dim), nn.Linear(a.ffn_dim, a.dim)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))

    def init_weights(self, **kwargs) -> None:
        for m in (self.fc1, self.fc2):
            nn.init.trunc_normal_(m.weight, mean=0.0, std=0.02)
            nn.init.zeros_(m.bias)


class EncoderLayer(Module):
    def __init__(self, a: Siglip2Config):
        super().__init__()
        self.layer_norm1 = nn.LayerNorm(a.dim, eps=a.layer_norm_eps)
        self.self_attn = _EncoderAttention(a)
        self.layer_norm2 = nn.LayerNorm(a.dim, eps=a.layer_norm_eps)
        self.mlp = _EncoderMLP(a)

    def forward(self, x, key_mask):
        x = x + self.self_attn(self.layer_norm1(x), key_mask)
        return x + self.mlp(self.layer_norm2(x))

    def init_weights(self, **kwargs) -> None:
        self.self_attn.init_weights()
        self.mlp.init_weights()
        self.layer_norm1.reset_parameters()
        self.layer_norm2.reset_parameters()


class VisionTransformer(Module):
    def __init__(self, a: Siglip2Config):
        super().__init__()
        self.args = a
        self.embeddings = VisionEmbeddings(a)
        self.layers = nn.ModuleDict({str(i): EncoderLayer(a) for i in range(a.n_layers)})
        self.post_layernorm = nn.LayerNorm(a.dim, eps=a.layer_norm_eps)

    def forward(self, pixels_nld, pixel_masks_nl, grid_hw):
        h = self.embeddings(pixels_nld, grid_hw)
        # padded images (no real patch) attend to everything to keep the softmax finite; their outputs are never used
        key_mask = pixel_masks_nl | ~pixel_masks_nl.any(dim=1, keepdim=True)
        for layer in self.layers.values():
            h = layer(h, key_mask)
        return self.post_layernorm(h)

    def init_weights(self, **kwargs) -> None:
        self.embeddings.init_weights()
        for layer in self.layers.values():
            layer.init_weights()
        self.post_layernorm.reset_parameters()


class Projector(Module):
    def __init__(self, in_dim: int, out_dim: int):
        super().__init__()
        self.w1, self.w2 = nn.Linear(in_dim, in_dim), nn.Linear(in_dim, out_dim)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)))

    def init_weights(self, **kwargs) -> None:
        for m in (self.w1, self.w2):
            nn.init.xavier_uniform_(m.weight)
            nn.init.zeros_(m.bias)


def _scatter_img_tokens(h_bsd, tokens_bs, i_nld, i_mask_nl, img_id: int):
    mask = (tokens_bs == img_id).unsqueeze(-1)
    flat = i_nld[i_mask_nl]
    assert flat.shape[0] == int(mask.sum()), (
        f"Different number of visual embeddings {flat.shape[0]} with placeholder in input token embeddings {int(mask.sum())}")
    return h_bsd.masked_scatter(mask.expand_as(h_bsd), flat.to(h_bsd.dtype))


class Llama3Siglip2Transformer(Llama3Model):
    @dataclass(kw_only=True, slots=True)
    class Config(Llama3Model.Config):
        encoder: Siglip2Config = field(default_factory=Siglip2Config)

    def __init__(self, config: Config):
        super().__init__(config)
        self.encoder = VisionTransformer(config.encoder)
        self.projector = Projector(config.encoder.dim, config.dim)

    def init_weights(self, **kwargs):
        super().init_weights(**kwargs)
        if self.encoder is not None:
            self.encoder.init_weights()
        if self.projector is not None:
            self.projector.init_weights()

    def get_attention_masks(self, input_batch, tokenizer, extra_inputs=None):
        masks = super().get_attention_masks(input_batch, tokenizer, extra_inputs)
        assert isinstance(masks, AttentionMasks)
        return {"llama3_masks": masks, "encoder_masks": None}

    def forward(self, tokens, pixel_values=None, grid_thw=None, special_tokens: SpecialTokens | None = None,
                attention_masks=None, positions=None):
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        if self.encoder is not None and pixel_values is not None:
            grid_hw = grid_thw[:, :, 1:]
            pixel_masks = (grid_hw != -1).all(dim=-1)
            img = self.projector(self.encoder(pixel_values.to(h.dtype), pixel_masks, grid_hw.clamp(min=0)))
            h = _scatter_img_tokens(h, tokens, img, pixel_masks, special_tokens.img_id)
        masks = attention_masks["llama3_masks"] if isinstance(attention_masks, dict) else attention_masks
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, masks, positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h

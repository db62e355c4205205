"""FLUX transformer <-> diffusers (Hugging Face ``FluxTransformer2DModel``) parameter names and layouts.

This model keeps the original layout of the architecture: one fused ``qkv`` projection per attention stream, one
``linear1`` per single-stream block that produces q, k, v and the MLP input together, and a final modulation that
stores (shift, scale). The diffusers checkpoint splits those projections into ``to_q`` / ``to_k`` / ``to_v`` (and
``add_*_proj`` for the text stream, ``proj_mlp`` for the single-stream MLP) and stores the final modulation as
(scale, shift). ``to_hf`` splits and swaps, ``from_hf`` concatenates and swaps back.
Parity: torchtitan/models/flux/model/state_dict_adapter.py (key map, fused-projection handling, final-layer swap)."""

from __future__ import annotations

import os
import re
from typing import Any

import torch

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter

# one-to-one names: ours -> diffusers
_PLAIN = {
    "img_in": "x_embedder",
    "txt_in": "context_embedder",
    "time_in.in_layer": "time_text_embed.timestep_embedder.linear_1",
    "time_in.out_layer": "time_text_embed.timestep_embedder.linear_2",
    "vector_in.in_layer": "time_text_embed.text_embedder.linear_1",
    "vector_in.out_layer": "time_text_embed.text_embedder.linear_2",
    "guidance_in.in_layer": "time_text_embed.guidance_embedder.linear_1",
    "guidance_in.out_layer": "time_text_embed.guidance_embedder.linear_2",
    "final_layer.linear": "proj_out",
    "final_layer.adaLN_modulation.1": "norm_out.linear",
    "double_blocks.{}.img_mod.lin": "transformer_blocks.{}.norm1.linear",
    "double_blocks.{}.txt_mod.lin": "transformer_blocks.{}.norm1_context.linear",
    "double_blocks.{}.img_attn.proj": "transformer_blocks.{}.attn.to_out.0",
    "double_blocks.{}.txt_attn.proj": "transformer_blocks.{}.attn.to_add_out",
    "double_blocks.{}.img_attn.norm.query_norm": "transformer_blocks.{}.attn.norm_q",
    "double_blocks.{}.img_attn.norm.key_norm": "transformer_blocks.{}.attn.norm_k",
    "double_blocks.{}.txt_attn.norm.query_norm": "transformer_blocks.{}.attn.norm_added_q",
    "double_blocks.{}.txt_attn.norm.key_norm": "transformer_blocks.{}.attn.norm_added_k",
    "double_blocks.{}.img_mlp.0": "transformer_blocks.{}.ff.net.0.proj",
    "double_blocks.{}.img_mlp.2": "transformer_blocks.{}.ff.net.2",
    "double_blocks.{}.txt_mlp.0": "transformer_blocks.{}.ff_context.net.0.proj",
    "double_blocks.{}.txt_mlp.2": "transformer_blocks.{}.ff_context.net.2",
    "single_blocks.{}.modulation.lin": "single_transformer_blocks.{}.norm.linear",
    "single_blocks.{}.linear2": "single_transformer_blocks.{}.proj_out",
    "single_blocks.{}.norm.query_norm": "single_transformer_blocks.{}.attn.norm_q",
    "single_blocks.{}.norm.key_norm": "single_transformer_blocks.{}.attn.norm_k",
}
# fused projections: ours -> the diffusers pieces, in concatenation order along dim 0
_FUSED = {
    "double_blocks.{}.img_attn.qkv": ["transformer_blocks.{}.attn.to_q", "transformer_blocks.{}.attn.to_k",
                                      "transformer_blocks.{}.attn.to_v"],
    "double_blocks.{}.txt_attn.qkv": ["transformer_blocks.{}.attn.add_q_proj", "transformer_blocks.{}.attn.add_k_proj",
                                      "transformer_blocks.{}.attn.add_v_proj"],
    "single_blocks.{}.linear1": ["single_transformer_blocks.{}.attn.to_q", "single_transformer_blocks.{}.attn.to_k",
                                 "single_transformer_blocks.{}.attn.to_v", "single_transformer_blocks.{}.proj_mlp"],
}
_SWAPPED = "final_layer.adaLN_modulation.1"
_PLAIN_REV = {v: k for k, v in _PLAIN.items()}
_PIECE_OF = {piece: (ours, i) for ours, pieces in _FUSED.items() for i, piece in enumerate(pieces)}


def _split_key(key: str) -> tuple[str, str | None, str]:
    """'double_blocks.3.img_attn.qkv.weight' -> ('double_blocks.{}.img_attn.qkv', '3', 'weight')."""
    stem, _, leaf = key.rpartition(".")
    m = re.search(r"blocks\.(\d+)\.", stem + ".")
    if m:
        return re.sub(r"blocks\.\d+", "blocks.{}", stem, count=1), m.group(1), leaf
    return stem, None, leaf


def _swap_halves(t: torch.Tensor) -> torch.Tensor:
    a, b = t.chunk(2, dim=0)
    return torch.cat((b, a), dim=0)


class FluxStateDictAdapter(StateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        if hf_assets_path and os.path.exists(os.path.join(hf_assets_path, "model_index.json")):
            hf_assets_path = os.path.join(hf_assets_path, "transformer")      # a full diffusers pipeline folder
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config

    def _hidden(self) -> int:
        return int(getattr(self.model_config, "hidden_size"))

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for key, value in state_dict.items():
            stem, layer, leaf = _split_key(key)
            if stem in _FUSED:
                h = self._hidden()
                sizes = [h, h, h] + ([value.shape[0] - 3 * h] if len(_FUSED[stem]) == 4 else [])
                for name, piece in zip(_FUSED[stem], torch.split(value, sizes, dim=0)):
                    out[f"{name.format(layer)}.{leaf}"] = piece.contiguous()
            elif stem in _PLAIN:
                v = _swap_halves(value) if stem == _SWAPPED else value
                name = _PLAIN[stem]
                out[f"{name.format(layer) if layer is not None else name}.{leaf}"] = v
            else:
                raise KeyError(f"no Hugging Face name for parameter {key}")
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        pieces: dict[str, list] = {}
        for key, value in hf_state_dict.items():
            stem, layer, leaf = _split_key(key)
            if stem in _PIECE_OF:
                ours, i = _PIECE_OF[stem]
                slot = pieces.setdefault(f"{ours.format(layer)}.{leaf}", [None] * len(_FUSED[ours]))
                slot[i] = value
            elif stem in _PLAIN_REV:
                ours = _PLAIN_REV[stem]
                v = _swap_halves(value) if ours == _SWAPPED else value
                out[f"{ours.format(layer) if layer is not None else ours}.{leaf}"] = v
            else:
                raise KeyError(f"no parameter for Hugging Face name {key}")
        for key, slot in pieces.items():
            if any(p is None for p in slot):
                raise KeyError(f"{key}: missing pieces of a fused projection")
            out[key] = torch.cat(slot, dim=0)
        return out

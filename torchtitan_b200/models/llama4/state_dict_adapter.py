"""Llama 4 <-> Hugging Face names (``language_model.*`` prefix). The grouped expert tensors are
stored transposed on the Hugging Face side and ``w1``/``w3`` are fused there as ``gate_up_proj``
along the last dimension; ``expert_bias`` has no Hugging Face counterpart.
Parity: torchtitan/models/llama4/state_dict_adapter.py:21-140."""

from __future__ import annotations

import re
from typing import Any

import torch

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter

_P = "language_model.model.layers.{}."
_FROM_HF = {
    "language_model.model.embed_tokens.weight": "tok_embeddings.weight",
    "language_model.model.norm.weight": "norm.weight",
    "language_model.lm_head.weight": "output.weight",
    _P + "self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
    _P + "self_attn.k_proj.weight": "layers.{}.attention.wk.weight",
    _P + "self_attn.v_proj.weight": "layers.{}.attention.wv.weight",
    _P + "self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
    _P + "input_layernorm.weight": "layers.{}.attention_norm.weight",
    _P + "post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
    _P + "feed_forward.router.weight": "layers.{}.moe.router.gate.weight",
    _P + "feed_forward.experts.down_proj": "layers.{}.moe.experts.w2",
    _P + "feed_forward.shared_expert.gate_proj.weight": "layers.{}.moe.shared_experts.w1.weight",
    _P + "feed_forward.shared_expert.down_proj.weight": "layers.{}.moe.shared_experts.w2.weight",
    _P + "feed_forward.shared_expert.up_proj.weight": "layers.{}.moe.shared_experts.w3.weight",
    _P + "feed_forward.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
    _P + "feed_forward.down_proj.weight": "layers.{}.feed_forward.w2.weight",
    _P + "feed_forward.up_proj.weight": "layers.{}.feed_forward.w3.weight",
}
_TO_HF = {v: k for k, v in _FROM_HF.items()}
_GATE_UP = _P + "feed_forward.experts.gate_up_proj"


def _split(key: str):
    if "layers" in key:
        return re.sub(r"(\d+)", "{}", key, count=1), re.search(r"\d+", key).group(0)
    return key, None


class Llama4StateDictAdapter(StateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        halves: dict[str, dict[str, Any]] = {}
        for key, value in state_dict.items():
            akey, layer = _split(key)
            if akey in ("layers.{}.moe.experts.w1", "layers.{}.moe.experts.w3"):
                halves.setdefault(layer, {})[akey[-2:]] = value.transpose(-1, -2)
            elif akey in _TO_HF:
                if akey == "layers.{}.moe.experts.w2":
                    value = value.transpose(-1, -2)
                out[_TO_HF[akey].format(layer) if layer is not None else _TO_HF[akey]] = value
        for layer, h in halves.items():
            out[_GATE_UP.format(layer)] = torch.cat((h["w1"], h["w3"]), dim=-1)
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for key, value in hf_state_dict.items():
            akey, layer = _split(key)
            if akey == _GATE_UP:
                w1, w3 = value.chunk(2, dim=-1)
                out[f"layers.{layer}.moe.experts.w1"] = w1.transpose(-1, -2)
                out[f"layers.{layer}.moe.experts.w3"] = w3.transpose(-1, -2)
            elif akey in _FROM_HF:
                if akey == _P + "feed_forward.experts.down_proj":
                    value = value.transpose(-1, -2)
                new = _FROM_HF[akey]
                out[new.format(layer) if layer is not None else new] = value
        return out

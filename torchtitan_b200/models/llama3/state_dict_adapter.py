"""Llama-3 <-> Hugging Face parameter names and layouts.

Parity: torchtitan/models/llama3/state_dict_adapter.py:18-144. HF stores ``q_proj`` / ``k_proj``
with each head's rotary pairs split into two halves (rotate-half convention) while this model
rotates adjacent pairs, so those two weights are permuted per head on the way in and out.
"""

from __future__ import annotations

import re
from typing import Any

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter

_TO_HF = {
    "tok_embeddings.weight": "model.embed_tokens.weight",
    "layers.{}.attention.wq.weight": "model.layers.{}.self_attn.q_proj.weight",
    "layers.{}.attention.wk.weight": "model.layers.{}.self_attn.k_proj.weight",
    "layers.{}.attention.wv.weight": "model.layers.{}.self_attn.v_proj.weight",
    "layers.{}.attention.wo.weight": "model.layers.{}.self_attn.o_proj.weight",
    "layers.{}.feed_forward.w1.weight": "model.layers.{}.mlp.gate_proj.weight",
    "layers.{}.feed_forward.w3.weight": "model.layers.{}.mlp.up_proj.weight",
    "layers.{}.feed_forward.w2.weight": "model.layers.{}.mlp.down_proj.weight",
    "layers.{}.attention_norm.weight": "model.layers.{}.input_layernorm.weight",
    "layers.{}.ffn_norm.weight": "model.layers.{}.post_attention_layernorm.weight",
    "norm.weight": "model.norm.weight",
    "output.weight": "lm_head.weight",
}
_FROM_HF = {v: k for k, v in _TO_HF.items()}
_FROM_HF["model.layers.{}.self_attn.rotary_emb.inv_freq"] = None


def _abstract(key: str) -> tuple[str, str | None]:
    m = re.search(r"\.(\d+)\.", key)
    if "layers" in key and m:
        return re.sub(r"(\d+)", "{}", key, count=1), m.group(1)
    return key, None


class Llama3StateDictAdapter(StateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config

    def _heads(self):
        a = self.model_config.layer.attention
        return a.n_heads, (a.n_kv_heads or a.n_heads)

    @staticmethod
    def _to_hf_layout(w, n_heads: int):
        """adjacent-pair rows -> half-split rows, per head."""
        d1, d2 = w.shape
        hd = d1 // n_heads
        return w.view(n_heads, hd // 2, 2, d2).transpose(1, 2).reshape(d1, d2)

    @staticmethod
    def _from_hf_layout(w, n_heads: int):
        d1, d2 = w.shape
        hd = d1 // n_heads
        return w.view(n_heads, 2, hd // 2, d2).transpose(1, 2).reshape(d1, d2)

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        nh, nkv = self._heads()
        out = {}
        for key, val in state_dict.items():
            akey, idx = _abstract(key)
            if akey not in _TO_HF:
                continue
            new = _TO_HF[akey]
            if idx is not None:
                new = new.format(idx)
            if akey.endswith("attention.wq.weight"):
                val = self._to_hf_layout(val, nh)
            elif akey.endswith("attention.wk.weight"):
                val = self._to_hf_layout(val, nkv)
            out[new] = val
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        nh, nkv = self._heads()
        out = {}
        for key, val in hf_state_dict.items():
            akey, idx = _abstract(key)
            if akey not in _FROM_HF or _FROM_HF[akey] is None:
                continue
            new = _FROM_HF[akey]
            if idx is not None:
                new = new.format(idx)
            if akey.endswith("q_proj.weight"):
                val = self._from_hf_layout(val, nh)
            elif akey.endswith("k_proj.weight"):
                val = self._from_hf_layout(val, nkv)
            out[new] = val
        return out

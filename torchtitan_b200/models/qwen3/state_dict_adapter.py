"""Qwen3 <-> Hugging Face names. Dense weights map one to one; grouped expert weights
``layers.N.moe.experts.w{1,2,3}`` ([E, out, in]) are split into / assembled from the per-expert
``mlp.experts.<e>.{gate,down,up}_proj.weight`` matrices.
Parity: torchtitan/models/qwen3/state_dict_adapter.py:25-190 and torchtitan/models/utils.py:19-386
(sharded grouped weights are split per local expert without gathering)."""

from __future__ import annotations

import re
from typing import Any

import torch

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter

_FROM_HF = {
    "model.embed_tokens.weight": "tok_embeddings.weight",
    "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
    "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.wk.weight",
    "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.wv.weight",
    "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
    "model.layers.{}.self_attn.q_norm.weight": "layers.{}.attention.q_norm.weight",
    "model.layers.{}.self_attn.k_norm.weight": "layers.{}.attention.k_norm.weight",
    "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
    "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
    "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
    "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
    "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
    "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
    "model.layers.{}.mlp.experts.{}.gate_proj.weight": "layers.{}.moe.experts.w1",
    "model.layers.{}.mlp.experts.{}.up_proj.weight": "layers.{}.moe.experts.w3",
    "model.layers.{}.mlp.experts.{}.down_proj.weight": "layers.{}.moe.experts.w2",
    "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
    "model.norm.weight": "norm.weight",
    "lm_head.weight": "output.weight",
}
_TO_HF = {v: k for k, v in _FROM_HF.items() if v is not None}


def _local(t):
    return t.to_local() if hasattr(t, "to_local") else t


class Qwen3StateDictAdapter(StateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config
        self._expert_meta: dict[str, Any] = {}

    def _expert_range(self, value) -> range:
        """Global expert ids held locally by a (possibly expert-sharded) grouped weight."""
        n_local = _local(value).shape[0]
        if hasattr(value, "device_mesh") and n_local != value.shape[0]:
            mesh, pls = value.device_mesh, value.placements
            start = 0
            for dim, pl in enumerate(pls):
                if getattr(pl, "dim", None) == 0 and pl.is_shard():
                    start += mesh.get_local_rank(dim) * n_local if len([p for p in pls if p.is_shard() and p.dim == 0]) == 1 else 0
            return range(start, start + n_local)
        return range(0, n_local)

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for key, value in state_dict.items():
            if "moe.experts" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                if akey not in _TO_HF:
                    continue
                layer = re.search(r"\d+", key).group(0)
                self._expert_meta[key] = value
                loc = _local(value)
                for i, e in enumerate(self._expert_range(value)):
                    out[_TO_HF[akey].format(layer, e)] = loc[i]
            elif "layers" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                if akey in _TO_HF:
                    out[_TO_HF[akey].format(re.search(r"\d+", key).group(0))] = value
            elif key in _TO_HF:
                if self.model_config.enable_weight_tying and key == "output.weight":
                    continue
                out[_TO_HF[key]] = value
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        experts: dict[str, dict[int, Any]] = {}
        if self.model_config.enable_weight_tying and "lm_head.weight" not in hf_state_dict and "model.embed_tokens.weight" in hf_state_dict:
            hf_state_dict = dict(hf_state_dict)
            hf_state_dict["lm_head.weight"] = hf_state_dict["model.embed_tokens.weight"]
        for key, value in hf_state_dict.items():
            if "mlp.experts" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=2)
                layer, e = re.findall(r"\d+", key)[:2]
                new = _FROM_HF[akey].format(layer)
                experts.setdefault(new, {})[int(e)] = value
            elif "layers" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                new = _FROM_HF.get(akey)
                if new is not None:
                    out[new.format(re.search(r"\d+", key).group(0))] = value
            elif key in _FROM_HF and _FROM_HF[key] is not None:
                out[_FROM_HF[key]] = value
        for new, per in experts.items():
            stacked = torch.stack([per[e] for e in sorted(per)], dim=0)
            meta = self._expert_meta.get(new)
            if meta is not None and hasattr(meta, "device_mesh"):
                from torch.distributed.tensor import DTensor

                stacked = DTensor.from_local(stacked, meta.device_mesh, meta.placements, run_check=False,
                                             shape=meta.shape, stride=meta.stride())
            out[new] = stacked
        return out

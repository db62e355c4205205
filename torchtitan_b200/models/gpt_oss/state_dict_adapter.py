"""gpt-oss <-> Hugging Face names. Expert tensors map as whole 3-D tensors (``*_blocks`` names on the
Hugging Face side); released checkpoints store them as MXFP4 (two e2m1 values per byte plus one E8M0
scale per 32 values), which :func:`dequantize_mxfp4` expands on load. Saving to MXFP4 is not offered.
Parity: torchtitan/models/gpt_oss/state_dict_adapter.py:17-118."""

from __future__ import annotations

import re
from typing import Any

import torch

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter

_L = "model.layers.{}."
_FROM_HF = {
    "model.embed_tokens.weight": "tok_embeddings.weight",
    **{_L + f"self_attn.{h}_proj.{p}": f"layers.{{}}.attention.w{h}.{p}" for h in "qkvo" for p in ("weight", "bias")},
    _L + "self_attn.sinks": "layers.{}.attention.sinks",
    _L + "input_layernorm.weight": "layers.{}.attention_norm.weight",
    _L + "post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
    _L + "mlp.experts.gate_up_proj_blocks": "layers.{}.moe.experts.mlp1_weight",
    _L + "mlp.experts.gate_up_proj_bias": "layers.{}.moe.experts.mlp1_bias",
    _L + "mlp.experts.down_proj_blocks": "layers.{}.moe.experts.mlp2_weight",
    _L + "mlp.experts.down_proj_bias": "layers.{}.moe.experts.mlp2_bias",
    _L + "mlp.router.weight": "layers.{}.moe.router.gate.weight",
    _L + "mlp.router.bias": "layers.{}.moe.router.gate.bias",
    "model.norm.weight": "norm.weight",
    "lm_head.weight": "output.weight",
}
_TO_HF = {v: k for k, v in _FROM_HF.items()}
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def dequantize_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """``blocks`` uint8 [..., G, 16] (low nibble first), ``scales`` uint8 [..., G] (E8M0, bias 127) -> [..., G*32]."""
    lut = torch.tensor(_E2M1, dtype=dtype, device=blocks.device)
    lo, hi = (blocks & 0x0F).long(), (blocks >> 4).long()
    vals = torch.stack((lut[lo], lut[hi]), dim=-1).flatten(-2)          # [..., G, 32]
    vals = vals * torch.exp2(scales.to(dtype) - 127).unsqueeze(-1)
    return vals.flatten(-2)


def _map(sd: dict[str, Any], table: dict[str, str]) -> dict[str, Any]:
    out = {}
    for key, value in sd.items():
        if "layers" in key:
            akey = re.sub(r"(\d+)", "{}", key, count=1)
            if akey in table:
                out[table[akey].format(re.search(r"\d+", key).group(0))] = value
        elif key in table:
            out[table[key]] = value
    return out


class GptOssStateDictAdapter(StateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config
        self.from_hf_map = dict(_FROM_HF)

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        return _map(state_dict, _TO_HF)

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        scales = {k[: -len("_scales")]: v for k, v in hf_state_dict.items() if k.endswith("_scales")}
        plain = {}
        for k, v in hf_state_dict.items():
            if k.endswith("_scales"):
                continue
            base = k[: -len("_blocks")] if k.endswith("_blocks") else None
            if base is not None and base in scales and v.dtype == torch.uint8:
                v = dequantize_mxfp4(v, scales[base])
            plain[k] = v
        return _map(plain, _FROM_HF)

    def get_hf_storage_reader(self, path: str, from_quantized: bool = False):
        from torch.distributed.checkpoint import HuggingFaceStorageReader

        if from_quantized:
            from torch.distributed.checkpoint.quantized_hf_storage import QuantizedHuggingFaceStorageReader

            return QuantizedHuggingFaceStorageReader(path=path, target_dtype=torch.float32, block_size=32, thread_count=4)
        return HuggingFaceStorageReader(path)

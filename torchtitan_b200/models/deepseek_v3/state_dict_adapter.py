"""DeepSeek-V3 <-> Hugging Face names; ``e_score_correction_bias`` is the expert bias; checkpoints stored as
block-scaled float8 (128 x 128 blocks with ``weight_scale_inv``) are dequantised on load.
Parity: torchtitan/models/deepseek_v3/state_dict_adapter.py:21-217."""

from __future__ import annotations

from typing import Any

import torch

from torchtitan_b200.models.utils import MoEStateDictAdapter, dequantize_block_fp8

_L = "model.layers.{}."


class DeepSeekV3StateDictAdapter(MoEStateDictAdapter):
    BLOCK_SIZE = 128

    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        m = {
            "model.embed_tokens.weight": "tok_embeddings.weight",
            _L + "self_attn.kv_a_proj_with_mqa.weight": "layers.{}.attention.wkv_a.weight",
            _L + "self_attn.kv_a_layernorm.weight": "layers.{}.attention.kv_norm.weight",
            _L + "self_attn.kv_b_proj.weight": "layers.{}.attention.wkv_b.weight",
            _L + "self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
            _L + "mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
            _L + "mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
            _L + "mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
            _L + "input_layernorm.weight": "layers.{}.attention_norm.weight",
            _L + "post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
            _L + "mlp.experts.{}.gate_proj.weight": "layers.{}.moe.experts.w1",
            _L + "mlp.experts.{}.up_proj.weight": "layers.{}.moe.experts.w3",
            _L + "mlp.experts.{}.down_proj.weight": "layers.{}.moe.experts.w2",
            _L + "mlp.gate.weight": "layers.{}.moe.router.gate.weight",
            _L + "mlp.shared_experts.gate_proj.weight": "layers.{}.moe.shared_experts.w1.weight",
            _L + "mlp.shared_experts.up_proj.weight": "layers.{}.moe.shared_experts.w3.weight",
            _L + "mlp.shared_experts.down_proj.weight": "layers.{}.moe.shared_experts.w2.weight",
            _L + "mlp.gate.e_score_correction_bias": "layers.{}.moe.expert_bias",
            "model.norm.weight": "norm.weight",
            "lm_head.weight": "output.weight",
        }
        if model_config.layer.attention.q_lora_rank != 0:
            m.update({
                _L + "self_attn.q_a_proj.weight": "layers.{}.attention.wq_a.weight",
                _L + "self_attn.q_a_layernorm.weight": "layers.{}.attention.q_norm.weight",
                _L + "self_attn.q_b_proj.weight": "layers.{}.attention.wq_b.weight",
            })
        else:
            m[_L + "self_attn.q_proj.weight"] = "layers.{}.attention.wq.weight"
        self.from_hf_map = m

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        # block-scaled float8 checkpoints: fold "<name>_scale_inv" into "<name>" first
        scales = {k: v for k, v in hf_state_dict.items() if k.endswith("_scale_inv")}
        if scales:
            plain = {}
            for k, v in hf_state_dict.items():
                if k.endswith("_scale_inv"):
                    continue
                s = scales.get(k + "_scale_inv")
                plain[k] = dequantize_block_fp8(v, s, self.BLOCK_SIZE) if s is not None else v
            hf_state_dict = plain
        return super().from_hf(hf_state_dict)

    def get_hf_storage_reader(self, path: str, from_quantized: bool = False):
        from torch.distributed.checkpoint import HuggingFaceStorageReader

        if from_quantized:
            from torch.distributed.checkpoint.quantized_hf_storage import QuantizedHuggingFaceStorageReader

            return QuantizedHuggingFaceStorageReader(path=path, target_dtype=torch.float32, block_size=self.BLOCK_SIZE,
                                                     thread_count=4)
        return HuggingFaceStorageReader(path)

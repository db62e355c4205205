"""Parameter / FLOP counting shared by model configs.

Parity: torchtitan/models/utils.py:389-514. FLOPs per token for training =
``6 * (N - N_embedding) + 6 * L * H * head_dims * S`` where ``head_dims`` is q-k plus v head
width (2*Dh for ordinary attention); for MoE only active expert parameters count.
"""

from __future__ import annotations

import torch.nn as nn


def _numel(p) -> int:
    return int(p.numel())


def get_dense_model_nparams_and_flops(model_config, model: nn.Module, n_heads: int, head_dims: int, seq_len: int):
    nparams = sum(_numel(p) for p in model.parameters())
    nparams_emb = sum(
        sum(_numel(p) for p in m.parameters()) for m in model.children() if isinstance(m, nn.Embedding)
    )
    flops = 6 * (nparams - nparams_emb) + 6 * model_config.n_layers * n_heads * head_dims * seq_len
    if getattr(model_config, "enable_weight_tying", False):
        # the reference's convention (torchtitan/models/utils.py:389-437): with tied embeddings the shared matrix is left
        # out of the reported parameter count and the output projection's matmul is not added to the FLOPs, so throughput
        # and MFU lines are comparable between the two frameworks
        nparams = nparams - nparams_emb
    return nparams, flops


def get_moe_model_nparams_and_flops(model_config, model: nn.Module, n_heads: int, head_dims: int, seq_len: int):
    emb = shared = routed = router = dense = 0
    for name, p in model.named_parameters():
        n = _numel(p)
        if "embedding" in name or "tok_embeddings" in name:
            emb += n
            dense += n
        elif "moe.shared_experts" in name:
            shared += n
        elif "moe.router" in name:
            router += n
        elif "moe.experts" in name:
            routed += n
        else:
            dense += n
    total = dense + shared + routed + router
    moe = model_config.layer.moe
    active = dense + shared + router + (routed * moe.top_k // moe.num_experts)
    flops = 6 * (active - emb) + 6 * model_config.n_layers * n_heads * head_dims * seq_len
    return total, flops


# ---- Hugging Face names for models with grouped experts ---------------------------------------

import re  # noqa: E402
from typing import Any  # noqa: E402

import torch  # noqa: E402

from torchtitan_b200.protocols.state_dict_adapter import StateDictAdapter  # noqa: E402


def _local(t):
    return t.to_local() if hasattr(t, "to_local") else t


class MoEStateDictAdapter(StateDictAdapter):
    """Name mapping driven by ``self.from_hf_map`` (Hugging Face name -> native name, ``{}`` for the
    layer and, in expert entries, the expert index). Grouped expert weights ``[E, out, in]`` are split
    into per-expert matrices on the way out and stacked on the way in. An expert-sharded (DTensor)
    grouped weight is split per *local* expert, never gathered, and the stacked result is wrapped
    back with the placements seen at ``to_hf`` time.
    Parity: torchtitan/models/utils.py:19-386."""

    from_hf_map: dict[str, str | None]

    def __init__(self, model_config, hf_assets_path: str | None):
        super().__init__(model_config, hf_assets_path)
        self.model_config = model_config
        self._expert_meta: dict[str, Any] = {}

    def _expert_range(self, value) -> range:
        n_local = _local(value).shape[0]
        if hasattr(value, "device_mesh") and n_local != value.shape[0]:
            mesh, start, stride = value.device_mesh, 0, value.shape[0]
            for dim, pl in enumerate(value.placements):
                if pl.is_shard() and pl.dim == 0:
                    stride //= mesh.size(dim)
                    start += mesh.get_local_rank(dim) * stride
            return range(start, start + n_local)
        return range(0, n_local)

    def _skip_to_hf(self, key: str) -> bool:
        return False

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        to_hf = {v: k for k, v in self.from_hf_map.items() if v is not None}
        out: dict[str, Any] = {}
        for key, value in state_dict.items():
            if self._skip_to_hf(key):
                continue
            if "moe.experts" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                if akey not in to_hf:
                    continue
                layer = re.search(r"\d+", key).group(0)
                self._expert_meta[key] = value
                loc = _local(value)
                for i, e in enumerate(self._expert_range(value)):
                    out[to_hf[akey].format(layer, e)] = loc[i]
            elif "layers" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                if akey in to_hf:
                    out[to_hf[akey].format(re.search(r"\d+", key).group(0))] = value
            elif key in to_hf:
                out[to_hf[key]] = value
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        experts: dict[str, dict[int, Any]] = {}
        for key, value in hf_state_dict.items():
            if "mlp.experts" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=2)
                if self.from_hf_map.get(akey) is None:
                    continue
                layer, e = re.findall(r"\d+", key)[:2]
                experts.setdefault(self.from_hf_map[akey].format(layer), {})[int(e)] = value
            elif "layers" in key:
                akey = re.sub(r"(\d+)", "{}", key, count=1)
                new = self.from_hf_map.get(akey)
                if new is not None:
                    out[new.format(re.search(r"\d+", key).group(0))] = value
            elif self.from_hf_map.get(key) is not None:
                out[self.from_hf_map[key]] = value
        for new, per in experts.items():
            stacked = torch.stack([per[e] for e in sorted(per)], dim=0)
            meta = self._expert_meta.get(new)
            if meta is not None and hasattr(meta, "device_mesh"):
                from torch.distributed.tensor import DTensor

                stacked = DTensor.from_local(stacked, meta.device_mesh, meta.placements, run_check=False,
                                             shape=meta.shape, stride=meta.stride())
            out[new] = stacked
        return out


def dequantize_block_fp8(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128,
                         dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``weight`` (float8, [N, K]) times its per-(block x block) inverse scale ([ceil(N/b), ceil(K/b)])."""
    n, k = weight.shape
    s = scale_inv.to(dtype).repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return weight.to(dtype) * s

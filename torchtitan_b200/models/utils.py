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
        sum(_numel(p) for p in m.parameters()) for m in model.modules() if isinstance(m, nn.Embedding)
    )
    flops = 6 * (nparams - nparams_emb) + 6 * model_config.n_layers * n_heads * head_dims * seq_len
    if getattr(model_config, "enable_weight_tying", False):
        # the tied output projection still does a matmul per token
        nparams = nparams  # parameters are shared, counted once by .parameters()
        flops += 6 * nparams_emb
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

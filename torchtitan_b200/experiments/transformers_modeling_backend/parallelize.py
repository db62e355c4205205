"""Activation checkpointing + FSDP/HSDP for wrapped Hugging Face decoders (one unit per decoder layer, one for
[norm, lm_head], one for the rest). Parity: torchtitan/experiments/transformers_modeling_backend/parallelize.py:41-400,
plus tensor parallel for the usual decoder layout (``self_attn.{q,k,v,o}_proj``, ``mlp.{gate,up,down}_proj``). Works on
the whole wrapper and on a pipeline stage alike (both expose ``layers`` / ``norm`` / ``output``); context parallel is
rejected in the model configuration."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.parallel import fsdp
from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy
from torchtitan_b200.tools.logging import logger


def _checkpoint_layer(layer: nn.Module) -> None:
    inner = layer.forward

    def forward(*args, **kwargs):
        if not torch.is_grad_enabled():
            return inner(*args, **kwargs)
        return checkpoint(inner, *args, use_reentrant=False, **kwargs)

    layer.forward = forward


class _CopyToTensorParallel(torch.autograd.Function):
    """Identity in forward; backward sums the input gradient over the group (each rank back-propagated through its own
    slice of the heads / hidden units)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def apply_tp_to_hf_decoder(model: nn.Module, tp_mesh) -> None:
    """Megatron-style tensor parallel over the module names most Hugging Face decoders share: q/k/v and gate/up projections
    are split by output features (whole heads), ``o_proj`` / ``down_proj`` by input features with a sum of the partial
    outputs. Hugging Face attention reshapes with ``-1`` heads, so it runs unchanged on its slice of the heads. Norms,
    embeddings and the output head stay replicated (activations are replicated: no sequence parallel here).
    Reference: torchtitan/experiments/transformers_modeling_backend/parallelize.py (its tensor-parallel plan)."""
    from torchtitan_b200.parallel.tp import _AllReduceSum, _shard_param, _wrap

    W, r, group = tp_mesh.size(), tp_mesh.get_local_rank(), tp_mesh.get_group()
    cfg = model.hf_config
    kv = getattr(cfg, "num_key_value_heads", None) or cfg.num_attention_heads
    if cfg.num_attention_heads % W or kv % W:
        raise ValueError(f"tensor parallel degree {W} must divide the head counts ({cfg.num_attention_heads} / {kv})")

    def region(mod, cols, rows):
        for name in cols + rows:
            if not hasattr(mod, name):
                raise NotImplementedError(f"tensor parallel for wrapped Hugging Face models expects a `{name}` projection in "
                                          f"{type(mod).__name__}")
        for name in cols:
            lin = getattr(mod, name)
            _shard_param(lin, "weight", 0, r, W, group, tp_mesh)
            if lin.bias is not None:
                _shard_param(lin, "bias", 0, r, W, group, tp_mesh)
            lin.out_features //= W
        for name in rows:
            lin = getattr(mod, name)
            if lin.bias is not None:
                raise NotImplementedError(f"{name}: a bias on a row-parallel projection is not supported")
            _shard_param(lin, "weight", 1, r, W, group, tp_mesh)
            lin.in_features //= W

        def fwd(inner, hidden_states, *a, **k):
            out = inner(_CopyToTensorParallel.apply(hidden_states, group), *a, **k)
            if isinstance(out, tuple):
                return (_AllReduceSum.apply(out[0], group),) + tuple(out[1:])
            return _AllReduceSum.apply(out, group)

        _wrap(mod, fwd)

    for layer in model.layers.values():
        region(layer.self_attn, ["q_proj", "k_proj", "v_proj"], ["o_proj"])
        region(layer.mlp, ["gate_proj", "up_proj"], ["down_proj"])
    logger.info(f"Applied tensor parallel (degree {W}) to the wrapped Hugging Face model")


_RING_NAME = "tt_ring_attention"
_rings: dict = {}


def _ring_attention_fn(module, query, key, value, attention_mask=None, dropout=0.0, scaling=None, **kwargs):
    """Attention function in the Hugging Face calling convention (``query`` [B, H, S, D], returns [B, S, H, D]) that runs
    this framework's context-parallel attention over the sequence shards."""
    ring = _rings[id(module.config)]
    out = ring(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), scale=scaling)
    return out.contiguous(), None


def apply_cp_to_hf_decoder(model: nn.Module, cp_mesh, rotate_method: str, load_balancer) -> None:
    """Context parallel for a wrapped decoder: the sequence is sharded head-tail by the trainer (inputs, labels, positions);
    rotary embeddings follow the explicit positions; every layer's attention goes through ``RingAttention`` (registered
    with Hugging Face's attention interface), and the model runs its parts directly instead of the top-level forward.
    Plain causal attention only. Reference: torchtitan/experiments/transformers_modeling_backend/parallelize.py (its
    context-parallel plan)."""
    from transformers.modeling_utils import AttentionInterface

    from torchtitan_b200.parallel.cp import RingAttention

    cfg = model.hf_config
    if getattr(cfg, "layer_types", None) and any(t != "full_attention" for t in cfg.layer_types):
        raise NotImplementedError("context parallel for wrapped models covers plain causal attention; this architecture "
                                  "mixes sliding-window layers")
    AttentionInterface.register(_RING_NAME, _ring_attention_fn)
    try:
        from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

        AttentionMaskInterface.register(_RING_NAME, sdpa_mask)
    except ImportError:
        pass
    ring = RingAttention(cp_mesh, rotate_method, load_balancer)
    from transformers import PretrainedConfig

    for c in {id(m.config): m.config for m in model.modules() if isinstance(getattr(m, "config", None), PretrainedConfig)}.values():
        c._attn_implementation = _RING_NAME
        _rings[id(c)] = ring
    model.__dict__["_call_parts_directly"] = True
    logger.info(f"Applied context parallel (degree {cp_mesh.size()}) to the wrapped Hugging Face model")


def parallelize_hf_transformers(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config,
                                ac_config, dump_folder: str):
    if parallel_dims.tp_enabled:
        apply_tp_to_hf_decoder(model, parallel_dims.get_mesh("tp"))
    if parallel_dims.cp_enabled:
        apply_cp_to_hf_decoder(model, parallel_dims.get_mesh("cp"), parallelism.context_parallel_rotate_method,
                               parallelism.context_parallel_load_balancer)
    layers = list(model.layers.values())
    if ac_config.mode == "full":
        for layer in layers:
            _checkpoint_layer(layer)
    elif ac_config.mode == "selective":
        every = int(ac_config.selective_ac_option) if str(ac_config.selective_ac_option).isdigit() else 1
        for i, layer in enumerate(layers):
            if every and (i + 1) % every == 0:
                _checkpoint_layer(layer)
    if parallel_dims.fsdp_enabled or parallel_dims.dp_replicate_enabled:
        mesh = parallel_dims.get_mesh(["dp_replicate", "fsdp"] if parallel_dims.dp_replicate_enabled and parallel_dims.fsdp_enabled
                                      else ("fsdp" if parallel_dims.fsdp_enabled else "dp_replicate"))
        mp = MixedPrecisionPolicy(param_dtype=TORCH_DTYPE_MAP[training.mixed_precision_param],
                                  reduce_dtype=TORCH_DTYPE_MAP[training.mixed_precision_reduce])
        if parallel_dims.fsdp_enabled:
            for layer in layers:
                fsdp.fully_shard(layer, mesh=mesh, mp_policy=mp)
            if not getattr(model.hf_config, "tie_word_embeddings", False):
                fsdp.fully_shard([model.norm, model.output], mesh=mesh, mp_policy=mp)
            fsdp.fully_shard(model, mesh=mesh, mp_policy=mp)
            logger.info("Applied FSDP to the wrapped Hugging Face model")
        else:
            fsdp.replicate(model, mesh=mesh, mp_policy=mp)
            logger.info("Applied DDP to the wrapped Hugging Face model")
    return model

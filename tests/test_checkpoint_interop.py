"""Checkpoint interchange with the reference, on CPU (gloo, 2 ranks, FSDP, fp32).

A DCP checkpoint of the model written by this framework (its ``ModelWrapper`` over the own FSDP runtime's DTensor
parameters) is loaded by the reference's ``ModelWrapper`` into the reference's own model under torch's ``fully_shard``,
and the loss of the next batch must be the same on both sides; then the reverse (the reference saves, this framework
loads). Both directions go through ``torch.distributed.checkpoint`` exactly as the two checkpoint managers do
(torchtitan/components/checkpoint.py:65-88 and ``dcp.save`` / ``dcp.load`` of the flattened model state).

The reference is taken from ``$TORCHTITAN_REFERENCE`` or the offline install under ``baseline/_ref``; skipped without it.
"""

import dataclasses
import os
import sys

import pytest
import torch

from dist_utils import run_ranks

_HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TORCHTITAN_REFERENCE") or os.path.join(os.path.dirname(_HERE), "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "torchtitan")), reason="reference not available")

SEQ, VOCAB = 128, 2048


def _batch(rank, seed):
    g = torch.Generator().manual_seed(seed * 100 + rank)
    x = torch.randint(0, VOCAB, (2, SEQ + 1), generator=g, dtype=torch.int64)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _build_ours(world, seed):
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"])
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=SEQ)
    torch.manual_seed(seed)
    model = cfg.build()
    model.init_weights()
    apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False)
    fsdp.materialize(model)
    return model


def _build_ref(world, seed):
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    from torchtitan.models.llama3 import llama3_configs

    cfg = llama3_configs["debugmodel"]
    layer = dataclasses.replace(cfg.layer, attention=dataclasses.replace(cfg.layer.attention, n_kv_heads=8))
    cfg = dataclasses.replace(cfg, layer=layer, rope=dataclasses.replace(cfg.rope, max_seq_len=SEQ))
    torch.manual_seed(seed)
    model = cfg.build()
    model.init_weights()
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    for blk in model.layers.values():
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    return model


def _loss(model, rank, seed, ce):
    import torch.distributed as dist

    x, y = _batch(rank, seed)
    with torch.no_grad():
        l = ce(model(x), y) / y.numel()
    dist.all_reduce(l)
    return float(l)


def _worker(rank, world, folder):
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp

    dist.init_process_group("gloo")
    from torchtitan_b200.components.checkpoint import ModelWrapper as OurWrapper
    from torchtitan_b200.components.loss import cross_entropy_loss as our_ce

    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.components.checkpoint import ModelWrapper as RefWrapper
    from torchtitan.components.loss import cross_entropy_loss as ref_ce

    out = {}
    # ---- this framework saves, the reference loads -------------------------------------------------------------
    ours = _build_ours(world, seed=11)
    ref = _build_ref(world, seed=22)                     # different weights before the load
    dcp.save(OurWrapper(ours).state_dict(), checkpoint_id=os.path.join(folder, "from_ours"))
    out["ref_before"] = _loss(ref, rank, 5, ref_ce)
    wrapper = RefWrapper(ref)
    sd = wrapper.state_dict()
    dcp.load(sd, checkpoint_id=os.path.join(folder, "from_ours"))
    wrapper.load_state_dict(sd)
    out["ours_a"], out["ref_a"] = _loss(ours, rank, 5, our_ce), _loss(ref, rank, 5, ref_ce)
    out["keys_equal"] = sorted(OurWrapper(ours).state_dict()) == sorted(RefWrapper(ref).state_dict())
    # ---- the reference saves, this framework loads -------------------------------------------------------------
    ref2 = _build_ref(world, seed=33)
    ours2 = _build_ours(world, seed=44)
    dcp.save(RefWrapper(ref2).state_dict(), checkpoint_id=os.path.join(folder, "from_ref"))
    w2 = OurWrapper(ours2)
    sd2 = w2.state_dict()
    dcp.load(sd2, checkpoint_id=os.path.join(folder, "from_ref"))
    w2.load_state_dict(sd2)
    out["ref_b"], out["ours_b"] = _loss(ref2, rank, 6, ref_ce), _loss(ours2, rank, 6, our_ce)
    return out


def test_model_checkpoints_load_across_the_two_frameworks(tmp_path):
    res = run_ranks(_worker, 2, str(tmp_path), tmp_path=tmp_path, timeout=900)
    o = res[0]
    assert o["keys_equal"]                                            # same fully-qualified names at the top level
    assert abs(o["ref_before"] - o["ours_a"]) > 1e-3                  # the load really changed the reference model
    assert abs(o["ours_a"] - o["ref_a"]) <= 1e-5 * abs(o["ours_a"]), o
    assert abs(o["ours_b"] - o["ref_b"]) <= 1e-5 * abs(o["ref_b"]), o

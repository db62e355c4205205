"""The NVLink peer-memory FSDP transport against the c10d (NCCL) transport on 2 GPUs: same seed, same batches, five
optimizer steps of two micro-batches each (gradient accumulation exercises the staging buffer's "read done" handshake).
The gradient shards of the first step (identical parameters on both sides) must agree to rounding; the losses of all
steps must agree loosely (Adam turns rounding-level gradient differences into different steps for near-zero
gradients, so later steps drift apart a little). A third run keeps the shards, their gradients and the optimizer state
in host memory (CPU offload): weights start from the same CPU initialisation, so its first-step gradients and its losses
are held to the same bounds. Skipped with fewer than two GPUs."""

import dataclasses

import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu

STEPS, MICRO, BATCH, SEQ = 5, 2, 2, 256


def _train(rank, world, fused: bool, offload: bool = False):
    import torch.distributed as dist

    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp

    class _Par:
        fused_fsdp_collectives = fused

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel"])
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=SEQ)
    torch.manual_seed(1234)
    with torch.device("cpu"):                         # CPU initialisation: the same weights with and without offload
        model = cfg.build()
    model.init_weights(buffer_device=torch.device("cuda"))
    if not offload:
        model.cuda()
    apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.bfloat16, reduce_dtype=torch.float32, pp_enabled=False,
               parallelism=_Par(), cpu_offload=offload)
    fsdp.materialize(model)
    units = fsdp.fsdp_units(model)
    transport = type(units[0].comm).__name__
    opt = OptimizersContainer.Config(lr=3e-3, beta1=0.9, beta2=0.95, weight_decay=0.1).build(model_parts=[model])
    g = torch.Generator().manual_seed(7 + rank)
    losses, grads = [], None
    for step in range(STEPS):
        opt.zero_grad()
        total = torch.zeros((), device="cuda")
        for _ in range(MICRO):
            x = torch.randint(0, cfg.vocab_size, (BATCH, SEQ + 1), generator=g).cuda()
            loss = cross_entropy_loss(model(x[:, :-1]), x[:, 1:]) / (BATCH * SEQ * MICRO * world)
            loss.backward()
            total += loss.detach()
        if step == 0:
            for u in units:
                u.wait_for_reduce()
            torch.cuda.synchronize()
            grads = [u.grad_shard_flat.detach().clone() for u in units if u.params]
        opt.step()
        dist.all_reduce(total)
        losses.append(total.item())
    torch.cuda.synchronize()
    errs = native.kernel_errors()
    comm_err = units[0].comm.errors() if hasattr(units[0].comm, "errors") else None
    return {"losses": losses, "grads": [t if offload else t.cpu() for t in grads], "transport": transport, "errs": errs,
            "comm_err": comm_err}


def _worker(rank, world):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    a = _train(rank, world, fused=True)
    b = _train(rank, world, fused=False)
    c = _train(rank, world, fused=False, offload=True)
    return a, b, c


def test_nvlink_transport_matches_c10d_with_gradient_accumulation(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = run_ranks(_worker, 2, tmp_path=tmp_path, timeout=900)
    for nv, c10, off in out:
        assert nv["transport"] == "NvlinkComm" and c10["transport"] == "C10dComm"
        assert not nv["errs"] and nv["comm_err"] is None
        # bf16 gradients cross the wire in both (NCCL reduces them in fp32 after a cast): same sums up to ordering
        assert abs(nv["losses"][0] - c10["losses"][0]) <= 1e-5 * abs(c10["losses"][0])
        for a, b in zip(nv["losses"], c10["losses"]):
            assert abs(a - b) <= 5e-3 * abs(b), (nv["losses"], c10["losses"])
        for ga, gb in zip(nv["grads"], c10["grads"]):
            scale = gb.abs().max().item() + 1e-12
            assert (ga - gb).abs().max().item() <= 5e-3 * scale, ((ga - gb).abs().max().item(), scale)
        assert nv["losses"][-1] < nv["losses"][0]
        # CPU offload: same collectives as the c10d run, gradients land in host memory, torch's AdamW steps on the CPU
        assert off["transport"] == "C10dComm" and not off["errs"]
        assert abs(off["losses"][0] - c10["losses"][0]) <= 1e-5 * abs(c10["losses"][0])
        for a, b in zip(off["losses"], c10["losses"]):
            assert abs(a - b) <= 5e-3 * abs(b), (off["losses"], c10["losses"])
        for ga, gb in zip(off["grads"], c10["grads"]):
            assert not ga.is_cuda
            scale = gb.abs().max().item() + 1e-12
            assert (ga - gb).abs().max().item() <= 1e-5 * scale

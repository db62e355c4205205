"""Tensor parallel (sequence parallel + loss parallel) against the single-process model on CPU."""

import dataclasses

import torch

from dist_utils import run_ranks


def _worker(rank, world, fsdp_too):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp
    from torchtitan_b200.parallel.tp import apply_tp_to_decoder, finalize_tp

    tp = 2
    pd = ParallelDims(dp_replicate=1, dp_shard=world // tp, cp=1, tp=tp, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    torch.manual_seed(7)
    ref = cfg.build()
    ref.init_weights()
    full = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    torch.manual_seed(100 + rank)
    x = torch.randint(0, cfg.vocab_size, (2, 65))
    # every rank of one TP group must see the same batch
    tp_mesh = pd.get_mesh("tp")
    dist.broadcast(x, src=dist.get_global_rank(tp_mesh.get_group(), 0), group=tp_mesh.get_group())
    inp, lab = x[:, :-1], x[:, 1:]

    model = cfg.build()
    model.load_state_dict(full)
    apply_tp_to_decoder(model, tp_mesh, loss_parallel=True)
    if fsdp_too:
        apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False)
        fsdp.materialize(model)
    finalize_tp(model)
    loss = cross_entropy_loss(model(inp), lab) / lab.numel()
    loss.backward()

    ref_loss = cross_entropy_loss(ref(inp), lab) / lab.numel()
    ref_loss.backward()
    out = {"loss": loss.item(), "ref": ref_loss.item()}
    # compare a column-parallel, a row-parallel and a replicated gradient (no FSDP case: local shards)
    if not fsdp_too:
        r = tp_mesh.get_local_rank()
        blk, rblk = model.layers["0"], ref.layers["0"]
        n = rblk.attention.wq.weight.shape[0] // tp
        out["wq"] = (blk.attention.wq.weight.grad - rblk.attention.wq.weight.grad[r * n : (r + 1) * n]).abs().max().item()
        k = rblk.attention.wo.weight.shape[1] // tp
        out["wo"] = (blk.attention.wo.weight.grad - rblk.attention.wo.weight.grad[:, r * k : (r + 1) * k]).abs().max().item()
        out["norm"] = (blk.attention_norm.weight.grad - rblk.attention_norm.weight.grad).abs().max().item()
        v = rblk.attention.wq.weight.shape[0]
        e = ref.tok_embeddings.weight.shape[0] // tp
        out["emb"] = (model.tok_embeddings.weight.grad - ref.tok_embeddings.weight.grad[r * e : (r + 1) * e]).abs().max().item()
    return out


def test_tp2_matches_single_process(tmp_path):
    res = run_ranks(_worker, 2, False, tmp_path=tmp_path)
    for o in res:
        assert abs(o["loss"] - o["ref"]) < 1e-5, o
        for k in ("wq", "wo", "norm", "emb"):
            assert o[k] < 1e-5, o


def test_tp2_fsdp2_loss_matches(tmp_path):
    res = run_ranks(_worker, 4, True, tmp_path=tmp_path)
    for o in res:
        assert abs(o["loss"] - o["ref"]) < 1e-5, o


def _moe_family_worker(rank, world, family):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.ep import apply_moe_ep_tp
    from torchtitan_b200.parallel.tp import apply_tp_to_decoder, finalize_tp

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    if family == "deepseek_v3":
        from torchtitan_b200.models.deepseek_v3 import deepseek_v3_configs

        cfg = dataclasses.replace(deepseek_v3_configs["debugmodel"], n_layers=2)
    else:
        from torchtitan_b200.models.gpt_oss import gptoss_configs

        cfg = dataclasses.replace(gptoss_configs["debugmodel"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=32)
    torch.manual_seed(11)
    ref = cfg.build()
    ref.init_weights(buffer_device=torch.device("cpu"))
    model = cfg.build()
    model.load_state_dict(ref.state_dict())
    model.freqs_cis = ref.freqs_cis.clone()
    apply_tp_to_decoder(model, pd.get_mesh("tp"), loss_parallel=True)
    apply_moe_ep_tp(model, pd, None)
    finalize_tp(model)
    x = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(5))
    inp, lab = x[:, :-1], x[:, 1:]
    masks = model.get_attention_masks(inp, None) if family == "gpt_oss" else None
    loss = cross_entropy_loss(model(inp, masks), lab) / lab.numel()
    loss.backward()
    ref_loss = cross_entropy_loss(ref(inp, masks), lab) / lab.numel()
    ref_loss.backward()
    out = {"loss": loss.item(), "ref": ref_loss.item()}
    g, rg = model.layers["1"].moe.router.gate.weight.grad, ref.layers["1"].moe.router.gate.weight.grad
    out["gate"] = (g - rg).abs().max().item()
    if family == "gpt_oss":
        out["wo_bias"] = (model.layers["0"].attention.wo.bias.grad - ref.layers["0"].attention.wo.bias.grad).abs().max().item()
    return out


def test_tp2_deepseek_mla_and_moe(tmp_path):
    for o in run_ranks(_moe_family_worker, 2, "deepseek_v3", tmp_path=tmp_path):
        assert abs(o["loss"] - o["ref"]) < 1e-5 and o["gate"] < 1e-5, o


def test_tp2_gpt_oss_sinks_biases_and_moe(tmp_path):
    for o in run_ranks(_moe_family_worker, 2, "gpt_oss", tmp_path=tmp_path):
        assert abs(o["loss"] - o["ref"]) < 1e-5 and o["gate"] < 1e-5 and o["wo_bias"] < 1e-5, o

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


def _ckpt_worker(rank, world, folder):
    """Save a model + optimizer under FSDP x TP, load it under plain FSDP (and back): every logical tensor must survive."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp

    dist.init_process_group("gloo")
    from torchtitan_b200.components.checkpoint import ModelWrapper
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp
    from torchtitan_b200.parallel.tp import apply_tp_to_decoder, finalize_tp

    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    torch.manual_seed(7)
    ref = cfg.build()
    ref.init_weights()
    full = {k: v.detach().clone() for k, v in ref.state_dict().items()}

    def build(tp, weights):
        pd = ParallelDims(dp_replicate=1, dp_shard=world // tp, cp=1, tp=tp, pp=1, ep=1, etp=1, world_size=world)
        m = cfg.build()
        if weights is not None:
            m.load_state_dict(weights)
        else:
            m.init_weights()
        if tp > 1:
            apply_tp_to_decoder(m, pd.get_mesh("tp"), loss_parallel=True)
        apply_fsdp(m, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False)
        fsdp.materialize(m)
        if tp > 1:
            finalize_tp(m)
        opt = OptimizersContainer.Config(name="AdamW", lr=1e-2, implementation="foreach").build(model_parts=[m])
        return pd, m, opt

    def step(pd, m, opt, seed):
        x = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(seed))
        from torchtitan_b200.components.loss import cross_entropy_loss

        loss = cross_entropy_loss(m(x[:, :-1]), x[:, 1:]) / x[:, 1:].numel()
        loss.backward()
        for u in fsdp.fsdp_units(m):
            u.wait_for_reduce()
        opt.step()
        opt.zero_grad()
        return loss.item()

    out = {}
    # (a) train one step under FSDP 2 x TP 2, save
    pd, m, opt = build(2, full)
    step(pd, m, opt, seed=1)                                    # same batch on every rank: dp ranks agree
    mw = ModelWrapper(m)
    sd = {"model": mw.state_dict(), "optimizer": opt.state_dict()}
    wq = sd["model"]["layers.0.attention.wq.weight"]
    out["wq_shape"] = tuple(wq.shape)
    saved_full = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).detach().clone() for k, v in sd["model"].items()}
    saved_opt = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).detach().clone()
                 for k, v in sd["optimizer"].items() if torch.is_tensor(v)}
    dcp.save(sd, checkpoint_id=folder)
    loss_a = step(pd, m, opt, seed=2)
    # (b) load under FSDP 4 (no TP) into a differently initialised model, continue
    torch.manual_seed(99)
    pd2, m2, opt2 = build(1, None)
    step(pd2, m2, opt2, seed=5)                                 # creates optimizer state to load into
    mw2 = ModelWrapper(m2)
    sd2 = {"model": mw2.state_dict(), "optimizer": opt2.state_dict()}
    dcp.load(sd2, checkpoint_id=folder)
    mw2.load_state_dict(sd2["model"])
    opt2.load_state_dict(sd2["optimizer"])
    got = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in mw2.state_dict().items()}
    out["model_diff"] = max((got[k].float() - saved_full[k].float()).abs().max().item() for k in saved_full)
    got_opt = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in opt2.state_dict().items() if torch.is_tensor(v)}
    out["opt_diff"] = max((got_opt[k].float() - saved_opt[k].float()).abs().max().item() for k in saved_opt)
    out["loss_diff"] = abs(step(pd2, m2, opt2, seed=2) - loss_a)
    # (c) and back: what FSDP 4 saves loads under FSDP 2 x TP 2
    dist.barrier()
    sd2 = {"model": mw2.state_dict(), "optimizer": opt2.state_dict()}
    want = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).detach().clone() for k, v in sd2["model"].items()}
    dcp.save(sd2, checkpoint_id=folder + "_b")
    torch.manual_seed(123)
    pd3, m3, opt3 = build(2, None)
    step(pd3, m3, opt3, seed=6)
    mw3 = ModelWrapper(m3)
    sd3 = {"model": mw3.state_dict(), "optimizer": opt3.state_dict()}
    dcp.load(sd3, checkpoint_id=folder + "_b")
    mw3.load_state_dict(sd3["model"])
    opt3.load_state_dict(sd3["optimizer"])
    got = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in mw3.state_dict().items()}
    out["back_diff"] = max((got[k].float() - want[k].float()).abs().max().item() for k in want)
    out["back_loss_diff"] = abs(step(pd3, m3, opt3, seed=3) - step(pd2, m2, opt2, seed=3))
    return out


def test_checkpoint_is_layout_independent_across_tp(tmp_path):
    """Reference: torchtitan/components/checkpoint.py (DCP state of DTensor parameters; loading on another parallel layout
    is the documented use)."""
    res = run_ranks(_ckpt_worker, 4, str(tmp_path / "ckpt"), tmp_path=tmp_path)
    for o in res:
        assert o["wq_shape"] == (256, 256), o                   # the full logical shape, not the tensor-parallel shard
        assert o["model_diff"] == 0 and o["opt_diff"] == 0 and o["back_diff"] == 0, o
        assert o["loss_diff"] < 1e-5 and o["back_loss_diff"] < 1e-5, o

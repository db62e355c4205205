"""Dense model families on CPU (forward shapes, determinism of initialisation, RoPE variants, attention masks, Hugging Face
state-dict adapters) and small utilities (model: the reference's tests/unit_tests/test_rope.py, test_module.py,
test_state_dict_adapter-style checks in scripts/checkpoint_conversion, test_utils)."""

import dataclasses
import gc

import os

import pytest
import torch


def _tiny(family: str, flavor: str):
    import importlib

    mod = importlib.import_module(f"torchtitan_b200.models.{family}")
    cfg = dataclasses.replace(getattr(mod, f"{family}_configs")[flavor])
    return cfg


@pytest.mark.parametrize("family,flavor", [("llama3", "debugmodel"), ("llama3", "debugmodel_gqa"), ("qwen3", "debugmodel")])
def test_dense_models_forward_backward_and_init_is_seeded(family, flavor):
    cfg = _tiny(family, flavor)
    torch.manual_seed(0)
    a = cfg.build()
    a.init_weights()
    torch.manual_seed(0)
    b = cfg.build()
    b.init_weights()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.equal(p, q), n
        assert torch.isfinite(p).all()
    tok = torch.randint(0, cfg.vocab_size, (2, 24))
    out = a(tok)
    assert out.shape == (2, 24, cfg.vocab_size)
    out.float().logsumexp(-1).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in a.parameters() if p.requires_grad)
    # causal: changing a later token leaves earlier logits untouched
    tok2 = tok.clone()
    tok2[:, -1] = (tok2[:, -1] + 1) % cfg.vocab_size
    assert torch.allclose(a(tok2)[:, :-1], out[:, :-1].detach(), atol=1e-5)


def test_model_flop_and_parameter_accounting():
    cfg = _tiny("llama3", "debugmodel")
    m = cfg.build()
    nparams, flops = cfg.get_nparams_and_flops(m, seq_len=128)
    assert nparams == sum(p.numel() for p in m.parameters())
    # 6 * (non-embedding parameters) + attention term
    emb = m.tok_embeddings.weight.numel()
    assert flops > 6 * (nparams - emb)


def test_rope_layouts_rotate_pairs_and_keep_norms():
    from torchtitan_b200.models.common.rope import RoPE, apply_rotary_emb

    for backend in ("complex", "cos_sin"):
        rope = RoPE(RoPE.Config(dim=16, max_seq_len=64, theta=10000.0, backend=backend))
        q = torch.randn(2, 10, 4, 16)
        k = torch.randn(2, 10, 2, 16)
        rq, rk = apply_rotary_emb(q, k, rope.cache, layout=rope.layout)
        assert rq.shape == q.shape and rk.shape == k.shape
        assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-4)      # rotations preserve length
        assert torch.allclose(rq[:, 0], q[:, 0], atol=1e-6)                     # position 0 is the identity
        # relative property: <R_m q, R_n k> depends on m - n only
        pos = torch.tensor([[3, 7]])
        pos2 = pos + 11
        a, b = torch.randn(1, 1, 1, 16), torch.randn(1, 1, 1, 16)
        qa, _ = apply_rotary_emb(a.expand(1, 2, 1, 16), a.expand(1, 2, 1, 16), rope.cache, positions=pos, layout=rope.layout)
        kb, _ = apply_rotary_emb(b.expand(1, 2, 1, 16), b.expand(1, 2, 1, 16), rope.cache, positions=pos, layout=rope.layout)
        qa2, _ = apply_rotary_emb(a.expand(1, 2, 1, 16), a.expand(1, 2, 1, 16), rope.cache, positions=pos2, layout=rope.layout)
        kb2, _ = apply_rotary_emb(b.expand(1, 2, 1, 16), b.expand(1, 2, 1, 16), rope.cache, positions=pos2, layout=rope.layout)
        d1 = (qa[0, 0, 0] * kb[0, 1, 0]).sum()
        d2 = (qa2[0, 0, 0] * kb2[0, 1, 0]).sum()
        assert torch.allclose(d1, d2, atol=1e-4)


def test_rope_scaling_variants_change_only_low_frequencies():
    from torchtitan_b200.models.common.rope import RoPE

    base = RoPE(RoPE.Config(dim=64, max_seq_len=128, theta=500000.0))
    llama = RoPE(RoPE.Config(dim=64, max_seq_len=128, theta=500000.0, scaling="llama", scaling_factor=8.0,
                             original_max_position_embeddings=64))
    f0, _ = base.inv_freq()
    f1, _ = llama.inv_freq()
    assert torch.allclose(f0[:2], f1[:2])                       # the fastest frequencies are untouched
    assert (f1[-4:] < f0[-4:]).all()                            # the slowest are stretched
    with pytest.raises(NotImplementedError):
        RoPE(RoPE.Config(dim=64, max_seq_len=128, backend="cos_sin", scaling="llama"))


def test_document_masks_block_attention_across_documents():
    from torchtitan_b200 import ops
    from torchtitan_b200.models.common.attention import create_varlen_metadata_for_document, document_ids, fixed_block_ids

    eos = 9
    tok = torch.tensor([[1, 2, eos, 3, 4, 5, eos, 6], [eos, 1, 2, 3, 4, eos, 5, 6]])
    ids = document_ids(tok, eos)
    assert ids.tolist() == [[0, 0, 0, 1, 1, 1, 1, 2], [0, 1, 1, 1, 1, 1, 2, 2]]
    meta = create_varlen_metadata_for_document(tok, eos)
    assert meta.cu_seqlens.tolist() == [0, 3, 7, 8, 9, 14, 16] and meta.max_seqlen == 5
    assert fixed_block_ids(1, 6, 4).tolist() == [[0, 0, 0, 0, 1, 1]]
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 8, 2, 16) for _ in range(3))
    out = ops.attention(q, k, v, causal=True, doc_ids=ids)
    # a document's outputs do not change when another document's values change
    v2 = v.clone()
    v2[0, :3] += 5.0
    out2 = ops.attention(q, k, v2, causal=True, doc_ids=ids)
    assert torch.allclose(out[0, 3:], out2[0, 3:], atol=1e-6) and not torch.allclose(out[0, :3], out2[0, :3])
    # sliding window: a key further back than the window has no influence
    w = ops.attention(q, k, v, causal=True, window=2)
    v3 = v.clone()
    v3[:, 0] += 5.0
    w3 = ops.attention(q, k, v3, causal=True, window=2)
    assert torch.allclose(w[:, 2:], w3[:, 2:], atol=1e-6)


@pytest.mark.parametrize("family,flavor", [("llama3", "debugmodel_gqa"), ("qwen3", "debugmodel")])
def test_hf_state_dict_adapter_round_trip(family, flavor):
    import importlib

    cfg = _tiny(family, flavor)
    m = cfg.build()
    m.init_weights()
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    mod = importlib.import_module(f"torchtitan_b200.models.{family}.state_dict_adapter")
    cls = next(getattr(mod, n) for n in dir(mod) if n.endswith("StateDictAdapter") and n != "StateDictAdapter" and "MoE" not in n)
    ad = cls(cfg, None)
    hf = ad.to_hf(sd)
    assert all(k.startswith(("model.", "lm_head.")) for k in hf), list(hf)[:5]
    assert any("self_attn.q_proj.weight" in k for k in hf) and any("mlp.down_proj.weight" in k for k in hf)
    back = ad.from_hf(hf)
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k]), k


def test_llama_rope_permutation_matches_hf_rotate_half():
    """The q/k projection rows are permuted between the interleaved layout used here and the half-rotated layout of
    Hugging Face checkpoints: scores must agree between the two conventions."""
    from torchtitan_b200.models.llama3.state_dict_adapter import Llama3StateDictAdapter

    n_heads, hd, dim = 2, 8, 16
    w = torch.randn(n_heads * hd, dim)
    hf = Llama3StateDictAdapter._to_hf_layout(w, n_heads)
    assert torch.equal(Llama3StateDictAdapter._from_hf_layout(hf, n_heads), w)
    x = torch.randn(5, dim)
    ours = (x @ w.t()).view(5, n_heads, hd // 2, 2)             # pairs (2i, 2i+1)
    theirs = (x @ hf.t()).view(5, n_heads, 2, hd // 2)           # halves (i, i + hd/2)
    assert torch.allclose(ours[..., 0], theirs[:, :, 0], atol=1e-6) and torch.allclose(ours[..., 1], theirs[:, :, 1], atol=1e-6)


def test_peak_flops_table_memory_monitor_and_gc():
    from torchtitan_b200.components.metrics import build_device_memory_monitor
    from torchtitan_b200.tools.utils import Color, GarbageCollection, NoColor, get_peak_flops

    assert get_peak_flops("NVIDIA B200") == 2.25e15
    assert get_peak_flops("NVIDIA H100 80GB HBM3") == 989e12
    assert get_peak_flops("some unknown device") == 312e12
    mon = build_device_memory_monitor()
    st = mon.get_peak_stats()
    assert st.max_reserved_gib >= 0 and 0 <= st.max_reserved_pct <= 100
    assert set(vars(NoColor)) >= {n for n in vars(Color) if not n.startswith("_")}
    was = gc.isenabled()
    try:
        h = GarbageCollection(gc_freq=2)
        assert not gc.isenabled()
        h.run(1)
        h.run(2)
        with pytest.raises(AssertionError):
            GarbageCollection(gc_freq=0)
    finally:
        if was:
            gc.enable()


def test_profiler_writes_traces_on_schedule_and_is_off_by_default(tmp_path):
    import glob

    from torchtitan_b200.tools.profiling import ProfilingConfig, maybe_enable_memory_snapshot, maybe_enable_profiling

    with maybe_enable_profiling(ProfilingConfig(), base_folder=str(tmp_path)) as prof:
        assert prof is None
    cfg = ProfilingConfig(enable_profiling=True, profile_freq=3, profiler_warmup=1, profiler_active=1)
    with maybe_enable_profiling(cfg, global_step=0, base_folder=str(tmp_path), leaf_folder="leaf") as prof:
        for _ in range(6):
            torch.randn(64, 64) @ torch.randn(64, 64)
            prof.step()
    traces = sorted(glob.glob(str(tmp_path / "profile_traces" / "iteration_*" / "leaf" / "rank0_trace.json")))
    assert len(traces) == 2, traces                           # one trace per period of profile_freq steps
    # repeat = 1 records a single cycle, skip_first delays it
    cfg = ProfilingConfig(enable_profiling=True, profile_freq=3, profiler_warmup=1, profiler_active=1, profiler_repeat=1,
                          profiler_skip_first=2, save_traces_folder="once")
    with maybe_enable_profiling(cfg, global_step=0, base_folder=str(tmp_path)) as prof:
        for _ in range(12):
            torch.randn(64, 64) @ torch.randn(64, 64)
            prof.step()
    assert sorted(os.listdir(tmp_path / "once")) == ["iteration_5"]
    with pytest.raises(AssertionError):
        with maybe_enable_profiling(ProfilingConfig(enable_profiling=True, profile_freq=2, profiler_warmup=3),
                                    base_folder=str(tmp_path)):
            pass
    with maybe_enable_memory_snapshot(ProfilingConfig(enable_memory_snapshot=True), base_folder=str(tmp_path)) as snap:
        assert snap is None or torch.cuda.is_available()      # memory snapshots need a CUDA device


def test_reference_names_of_building_blocks_and_mask_functions():
    """Names that code written against the reference imports: the parallelize steps of every family, the mask functions
    of the common attention module (checked against the documents / window they describe), loader and
    fault-tolerance exports."""
    import importlib

    from torch.nn.attention.flex_attention import and_masks, create_mask

    wanted = {f"torchtitan_b200.models.{f}.parallelize": ["apply_ac", "apply_fsdp", "apply_compile", "apply_non_moe_tp",
                                                          "apply_moe_ep_tp", "disable_fsdp_gradient_division"]
              for f in ("llama3", "llama4", "qwen3", "deepseek_v3", "gpt_oss")}
    wanted.update({
        "torchtitan_b200.models.flux.parallelize": ["apply_ac", "apply_fsdp", "parallelize_flux"],
        "torchtitan_b200.models.common": ["MoE", "apply_rotary_emb_cos_sin", "apply_rotary_emb_complex", "create_attention_mask",
                                          "get_causal_mask_mod", "get_document_mask_mod", "get_fixed_block_mask_mod",
                                          "get_sliding_window_mask_mod", "create_varlen_metadata_for_document"],
        "torchtitan_b200.models.common.moe.kernels": ["generate_permute_indices", "fill_indices_wrapper"],
        "torchtitan_b200.components.quantization.module_utils": ["capture_module_attrs", "inject_module_protocol",
                                                                 "verify_module_protocol"],
        "torchtitan_b200.distributed": ["ParallelDims", "utils", "parallel_dims"],
        "torchtitan_b200.distributed.utils": ["set_determinism", "clip_grad_norm_", "dist_mean", "init_distributed"],
        "torchtitan_b200.distributed.tensor_parallel": ["maybe_enable_async_tp"],
        "torchtitan_b200.distributed.activation_checkpoint": ["apply_ac"],
        "torchtitan_b200.experiments.ft": ["has_torchft", "maybe_semi_sync_training"],
        "torchtitan_b200.experiments.ft.llama3": ["model_registry"],
        "torchtitan_b200.experiments.vlm": ["HuggingFaceMultiModalDataLoader"],
        "torchtitan_b200.experiments.vlm.configs": ["MultiModalTrainerConfig"],
        "torchtitan_b200.models.flux.configs": ["Encoder", "Validation", "Inference"],
    })
    for module, names in wanted.items():
        mod = importlib.import_module(module)
        for n in names:
            assert getattr(mod, n, None) is not None, f"{module}.{n}"
    from torchtitan_b200.models.common import (get_causal_mask_mod, get_document_mask_mod, get_fixed_block_mask_mod,
                                               get_sliding_window_mask_mod)

    x = torch.tensor([[5, 1, 7, 7, 1, 3, 4, 9]])                    # three documents ending with token 1
    doc = torch.tensor([0, 0, 1, 1, 1, 2, 2, 2])
    i = torch.arange(8)
    causal = i[:, None] >= i[None, :]
    got = create_mask(and_masks(get_causal_mask_mod(), get_document_mask_mod(x, 1), get_sliding_window_mask_mod(2)), 1, 1, 8, 8,
                      device="cpu")[0, 0]
    assert torch.equal(got, causal & (doc[:, None] == doc[None, :]) & (i[:, None] - i[None, :] < 2))
    blocks = create_mask(and_masks(get_causal_mask_mod(), get_fixed_block_mask_mod(4)), 1, 1, 8, 8, device="cpu")[0, 0]
    assert torch.equal(blocks, causal & (i[:, None] // 4 == i[None, :] // 4))
    # a module swapped for another class keeps the Module protocol and its saved attributes
    from torchtitan_b200.components.quantization.module_utils import (capture_module_attrs, inject_module_protocol,
                                                                       verify_module_protocol)
    from torchtitan_b200.models.common.linear import Linear

    class Foreign(torch.nn.Linear):
        pass

    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2))
    net[0].tag, net[1].tag = "first", "second"
    saved = capture_module_attrs(net, ["tag"])
    net[0], net[1] = Foreign(4, 4), Foreign(4, 2)
    with pytest.raises(RuntimeError, match="do not satisfy"):
        verify_module_protocol(net, Foreign, Linear)
    inject_module_protocol(net, Linear, saved)
    verify_module_protocol(net, Foreign, Linear)
    assert (net[0].tag, net[1].tag) == ("first", "second") and type(net[0]) is type(net[1]) and isinstance(net[0], Foreign)
    with pytest.raises(RuntimeError, match="should not be constructed directly"):
        type(net[0])(4, 4)


def test_token_group_padding_wrapper_and_alignment_floor():
    """``indices_padding_wrapper`` hands a per-expert function padded, expert-major groups and restores the row order; the
    alignment floor set by converters raises what the dispatchers pad to."""
    from torchtitan_b200.models.common.moe import utils as u
    from torchtitan_b200.models.common.moe.moe import group_alignment

    torch.manual_seed(0)
    E, D = 3, 4
    w1, w2, w3 = torch.randn(E, 5, D), torch.randn(E, D, 5), torch.randn(E, 5, D)
    counts = torch.tensor([2, 0, 3, 1, 4, 0], dtype=torch.int32)            # 2 source ranks x 3 local experts
    x = torch.randn(int(counts.sum()), D)
    seen = {}

    def per_expert(w1, w2, w3, xp, c):
        seen["counts"] = c.tolist()
        out, off = torch.zeros(xp.shape[0], D), 0
        for e, n in enumerate(c.tolist()):
            h = xp[off:off + n]
            out[off:off + n] = (torch.nn.functional.silu(h @ w1[e].t()) * (h @ w3[e].t())) @ w2[e].t()
            off += n
        return out

    got = u.indices_padding_wrapper(per_expert)(w1, w2, w3, x, counts)
    owner = torch.repeat_interleave(torch.arange(6) % 3, counts.long())
    want = torch.stack([(torch.nn.functional.silu(x[i] @ w1[e].t()) * (x[i] @ w3[e].t())) @ w2[e].t()
                        for i, e in enumerate(owner.tolist())])
    assert torch.allclose(got, want, atol=1e-5) and seen["counts"] == [8, 8, 8]     # 3, 4, 3 rows padded to the alignment
    try:
        u.set_token_group_alignment_size_m(32)
        assert u.get_mxfp8_pad_multiple() == 32 and u.maybe_align_num_tokens_for_mxfp8(33) == 64
        assert group_alignment(object(), 8) == 32 and group_alignment(object(), 64) == 64
        with pytest.raises(ValueError):
            u.set_token_group_alignment_size_m(12)
    finally:
        u.set_token_group_alignment_size_m(8)
    assert u.get_mxfp8_pad_multiple() is None and group_alignment(object(), 8) == 8

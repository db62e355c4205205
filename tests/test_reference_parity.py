"""Loss parity with the reference implementation on CPU (gloo, 2 ranks, FSDP, fp32).

Config: Llama-3 debug model with 8 KV heads (dim 256, 6 layers, 16 heads, FFN 768, vocab 2048,
RoPE theta 500000), local batch 2 x seq 512 of uniform tokens from seed 0, AdamW lr 8e-4
betas (0.9, 0.95) wd 0.1, warmup 2 of 10 steps. Both sides start from identical weights; ours
runs this framework's model + FSDP runtime + optimizer container + LR schedule, the other side
runs the reference's model code with torch's ``fully_shard``, ``AdamW`` and the reference's own
``LRSchedulersContainer``. Losses must agree to rtol 1e-4 at every step. A second test compares
the learning-rate multipliers of the two schedulers step by step.

The reference is taken from ``$TORCHTITAN_REFERENCE`` (a checkout) or from the offline install
under ``baseline/_ref``; without either the tests are skipped.
"""

import dataclasses
import os
import sys

import pytest
import torch

from dist_utils import run_ranks

_HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TORCHTITAN_REFERENCE") or os.path.join(os.path.dirname(_HERE), "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "torchtitan")), reason="reference tree not mounted")

STEPS, WARMUP, BATCH, SEQ, VOCAB = 10, 2, 2, 512, 2048


def _batches(rank: int):
    g = torch.Generator().manual_seed(0 + rank)
    for _ in range(STEPS):
        x = torch.randint(0, VOCAB, (BATCH, SEQ + 1), generator=g, dtype=torch.int64)
        yield x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _ours(rank, world, init_state):
    import torch.distributed as dist

    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp
    from torchtitan_b200.parallel.utils import clip_grad_norm_

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"])
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=SEQ)
    torch.manual_seed(1234)
    model = cfg.build()
    model.init_weights()
    if init_state is not None:
        model.load_state_dict(init_state)
    full_state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False)
    fsdp.materialize(model)
    opt = OptimizersContainer.Config(lr=8e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, implementation="foreach").build(model_parts=[model])
    sched = LRSchedulersContainer.Config(warmup_steps=WARMUP).build(optimizers=opt, training_steps=STEPS)
    losses = []
    for x, y in _batches(rank):
        opt.zero_grad()
        ntok = torch.tensor(float(y.numel()))
        dist.all_reduce(ntok)
        loss = cross_entropy_loss(model(x), y) / ntok
        loss.backward()
        clip_grad_norm_(list(model.parameters()), 1.0)
        opt.step()
        sched.step()
        l = loss.detach().clone()
        dist.all_reduce(l)
        losses.append(l.item())
    return losses, full_state


def _reference(rank, world, init_state):
    sys.path.insert(0, REF)
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    from torchtitan.components.loss import cross_entropy_loss
    from torchtitan.models.llama3 import llama3_configs

    cfg = llama3_configs["debugmodel"]
    layer = dataclasses.replace(cfg.layer, attention=dataclasses.replace(cfg.layer.attention, n_kv_heads=8))
    cfg = dataclasses.replace(cfg, layer=layer, rope=dataclasses.replace(cfg.rope, max_seq_len=SEQ))
    model = cfg.build()
    model.init_weights()
    model.load_state_dict(init_state)
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    for blk in model.layers.values():
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    # torch's FSDP averages gradients over ranks (its "no division" mode needs PREMUL_SUM, which
    # gloo lacks); multiplying the loss by the world size (exact in fp32) gives the same sum.
    from torchtitan.components.lr_scheduler import LRSchedulersContainer as RefSchedulers

    opt = torch.optim.AdamW(model.parameters(), lr=8e-4, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    sched = RefSchedulers.Config(warmup_steps=WARMUP).build(optimizers=[opt], training_steps=STEPS)
    losses = []
    for x, y in _batches(rank):
        opt.zero_grad()
        ntok = torch.tensor(float(y.numel()))
        dist.all_reduce(ntok)
        loss = cross_entropy_loss(model(x), y) / ntok
        (loss * world).backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        l = loss.detach().clone()
        dist.all_reduce(l)
        losses.append(l.item())
    return losses


def _both(rank, world):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    ours, state = _ours(rank, world, None)
    ref = _reference(rank, world, state)
    return ours, ref


def test_loss_matches_reference_fsdp2_cpu(tmp_path):
    out = run_ranks(_both, 2, tmp_path=tmp_path, timeout=900)
    ours, ref = out[0]
    assert len(ours) == STEPS
    for a, b in zip(ours, ref):
        assert abs(a - b) <= 1e-4 * abs(b), (ours, ref)
    assert ours[-1] < ours[0]


@pytest.mark.parametrize("kind", ["linear", "sqrt", "cosine"])
@pytest.mark.parametrize("decay_ratio,floor", [(None, 0.0), (0.3, 0.0), (0.25, 0.1), (None, 0.2)])
def test_lr_multipliers_match_the_reference_scheduler_step_by_step(kind, decay_ratio, floor):
    """Same multiplier at every step as the reference's own ``LRSchedulersContainer`` (built through its Config)."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.components.lr_scheduler import LRSchedulersContainer as RefSchedulers

    from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer

    total, warmup = 100, 10
    kw = dict(warmup_steps=warmup, decay_ratio=decay_ratio, decay_type=kind, min_lr_factor=floor)

    def curve(container_cls):
        opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
        sched = container_cls.Config(**kw).build(optimizers=[opt], training_steps=total)
        out = []
        for _ in range(total):
            out.append(opt.param_groups[0]["lr"])
            opt.step()
            sched.step()
        return out

    ours, ref = curve(LRSchedulersContainer), curve(RefSchedulers)
    assert ours == pytest.approx(ref, rel=1e-12, abs=1e-15)
    assert ours[0] == pytest.approx(1 / warmup) and ours[warmup - 1] == pytest.approx(1.0)


def _no_grouped(cfg):
    """Copy of a model configuration tree with every ``use_grouped_mm`` switched off: the reference's grouped path pads
    token groups with a Triton kernel, its per-expert loop runs on the CPU."""
    if dataclasses.is_dataclass(cfg) and not isinstance(cfg, type):
        changes = {}
        for f in dataclasses.fields(cfg):
            if not f.init:
                continue
            v = getattr(cfg, f.name, None)
            if f.name == "use_grouped_mm":
                changes[f.name] = False
            elif dataclasses.is_dataclass(v) and not isinstance(v, type):
                changes[f.name] = _no_grouped(v)
            elif isinstance(v, list) and v and dataclasses.is_dataclass(v[0]):
                changes[f.name] = [_no_grouped(x) for x in v]
        return dataclasses.replace(cfg, **changes) if changes else cfg
    return cfg


def _dense_flex_attention(q, k, v, block_mask=None, scale=None, enable_gqa=False, return_lse=False):
    """Stand-in for the reference's compiled flex attention on the CPU: the plain definition of attention under the
    reference's own ``mask_mod`` (taken from the block mask it built), with the log-sum-exp it asks for."""
    from torch.nn.attention.flex_attention import create_mask

    B, H, S, D = q.shape
    if k.shape[1] != H:
        k, v = k.repeat_interleave(H // k.shape[1], 1), v.repeat_interleave(H // v.shape[1], 1)
    s = (q.float() @ k.float().transpose(-1, -2)) * (scale if scale is not None else D ** -0.5)
    if block_mask is not None:
        s = s.masked_fill(~create_mask(block_mask.mask_mod, B, 1, S, k.shape[2], device="cpu"), float("-inf"))
    out = (torch.softmax(s, -1) @ v.float()).to(q.dtype)
    return (out, torch.logsumexp(s, -1)) if return_lse else out


@pytest.mark.parametrize("family,flavor", [("llama3", "debugmodel"), ("qwen3", "debugmodel"), ("qwen3", "debugmodel_moe"),
                                           ("deepseek_v3", "debugmodel"), ("gpt_oss", "debugmodel"), ("llama4", "debugmodel")])
def test_model_families_match_the_reference_models(family, flavor, monkeypatch):
    """Same parameter names and shapes as the reference's model of the family; with this framework's weights loaded into
    the reference's own model code, logits and every parameter gradient agree (fp32, CPU): dense and MoE Qwen3 (q / k
    norms, top-k softmax routing), DeepSeek-V3 (multi-head latent attention, sigmoid routing with shared experts),
    GPT-OSS (sinks, alternating sliding-window layers, biased experts with the clamped activation) and Llama 4 (layers
    without rotary embedding, attention in fixed blocks, shared expert). The last two build document masks from
    end-of-sequence tokens, planted here, over sequences longer than the window and the block; the reference's compiled
    flex attention (GPU only) is replaced by the definition of attention under the reference's own mask function."""
    import importlib

    if REF not in sys.path:
        sys.path.insert(0, REF)
    masked = family in ("gpt_oss", "llama4")
    if masked:
        from torch.nn.attention.flex_attention import create_block_mask

        import torchtitan.models.common.attention as ref_attention

        monkeypatch.setattr(ref_attention.FlexAttentionWrapper, "_compiled_flex_attn", staticmethod(_dense_flex_attention))
        monkeypatch.setattr(ref_attention, "_compiled_create_block_mask",
                            lambda *a, **k: create_block_mask(*a, **{**k, "device": "cpu"}))
    histc = torch.histc
    # the reference counts tokens per expert with histc on integer indices, which the CPU kernel does not take
    monkeypatch.setattr(torch, "histc", lambda x, *a, **k: histc(x.float(), *a, **k).to(x.dtype))

    def configs(mod):
        return getattr(mod, next(a for a in dir(mod) if a.endswith("_configs")))

    ours_cfg = _no_grouped(configs(importlib.import_module(f"torchtitan_b200.models.{family}"))[flavor])
    ref_cfg = _no_grouped(configs(importlib.import_module(f"torchtitan.models.{family}"))[flavor])
    torch.manual_seed(0)
    ours = ours_cfg.build()
    ours.init_weights()
    ref = ref_cfg.build()
    state = ours.state_dict()
    ref_state = ref.state_dict()
    assert set(state) == set(ref_state)
    assert all(state[k].shape == ref_state[k].shape for k in state)
    ref.load_state_dict(state)
    if hasattr(ref, "freqs_cis") and hasattr(ours, "freqs_cis") and ref.freqs_cis.shape == ours.freqs_cis.shape:
        ref.freqs_cis = ours.freqs_cis.clone()                     # non-persistent buffer: not part of the state dict
    else:
        with torch.no_grad():
            ref.init_weights(buffer_device=torch.device("cpu")) if family != "llama3" else ref.init_weights()
        ref.load_state_dict(state)
    x = torch.randint(8, ours_cfg.vocab_size, (2, 321 if masked else 65))
    kw_ours, kw_ref = {}, {}
    if masked:
        class _Tok:
            eos_id = 3

        x[0, [40, 41, 170]] = _Tok.eos_id                          # three documents in row 0 (one of a single token), two in row 1
        x[1, 299] = _Tok.eos_id
    inp, lab = x[:, :-1], x[:, 1:]
    if masked:
        kw_ours = {"attention_masks": ours.get_attention_masks(inp, _Tok())}
        kw_ref = {"attention_masks": ref.get_attention_masks(inp, _Tok())}
    lo, lr = ours(inp, **kw_ours), ref(inp, **kw_ref)
    assert (lo - lr).abs().max().item() < 2e-5 * max(lr.abs().max().item(), 1.0)
    torch.nn.functional.cross_entropy(lo.flatten(0, 1).float(), lab.flatten()).backward()
    torch.nn.functional.cross_entropy(lr.flatten(0, 1).float(), lab.flatten()).backward()
    ref_grads = dict(ref.named_parameters())
    for name, p in ours.named_parameters():
        g, w = p.grad, ref_grads[name].grad
        assert (g is None) == (w is None), name
        if g is not None:
            assert (g - w).abs().max().item() <= 1e-4 * max(w.abs().max().item(), 1e-6) + 1e-7, name


@pytest.mark.parametrize("family,flavor", [("llama3", "debugmodel"), ("qwen3", "debugmodel"), ("qwen3", "debugmodel_moe"),
                                           ("deepseek_v3", "debugmodel"), ("gpt_oss", "debugmodel"), ("llama4", "debugmodel")])
def test_hf_state_dict_adapters_match_the_reference_adapters(family, flavor):
    """The Hugging Face export of a model's state (names, shapes, values: fused / split projections, expert stacking,
    permuted rotary layouts) equals what the reference's adapter writes, and reading the reference's export back gives
    what the reference's own adapter reads. Llama 4: the reference's export leaves out the dense layers' feed-forward
    weights; this framework writes them, everything the reference writes is equal."""
    import importlib

    if REF not in sys.path:
        sys.path.insert(0, REF)

    def first(mod, suffix):
        return getattr(mod, next(a for a in dir(mod) if a.endswith(suffix)))

    om, rm = importlib.import_module(f"torchtitan_b200.models.{family}"), importlib.import_module(f"torchtitan.models.{family}")
    ours_cfg, ref_cfg = first(om, "_configs")[flavor], first(rm, "_configs")[flavor]
    ours_adapter, ref_adapter = first(om, "StateDictAdapter")(ours_cfg, None), first(rm, "StateDictAdapter")(ref_cfg, None)
    torch.manual_seed(0)
    model = ours_cfg.build()
    model.init_weights()
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    ours_hf, ref_hf = ours_adapter.to_hf(dict(state)), ref_adapter.to_hf(dict(state))
    if family == "llama4":
        assert set(ref_hf) <= set(ours_hf)
    else:
        assert set(ref_hf) == set(ours_hf)
    for k, v in ref_hf.items():
        assert ours_hf[k].shape == v.shape and torch.equal(ours_hf[k], v), k
    back_ours, back_ref = ours_adapter.from_hf(dict(ref_hf)), ref_adapter.from_hf(dict(ref_hf))
    assert set(back_ours) == set(back_ref)
    for k, v in back_ref.items():
        assert torch.equal(back_ours[k], v) and torch.equal(v, state[k]), k


def _config_tree(cls_or_obj, prefix="", out=None, depth=0):
    out = {} if out is None else out
    if depth > 6:
        return out
    for f in dataclasses.fields(cls_or_obj):
        value = None
        if f.default is not dataclasses.MISSING:
            value = f.default
        elif f.default_factory is not dataclasses.MISSING:
            try:
                value = f.default_factory()
            except Exception:
                value = None
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            _config_tree(value, prefix + f.name + ".", out, depth + 1)
        else:
            out[prefix + f.name] = value
    return out


def test_every_job_option_of_the_reference_exists_with_the_same_default():
    """The trainer's configuration tree (what ``--section.option`` flags and job configurations address): no option of
    the reference is missing and none has another default; options that only exist here are additions."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.trainer import Trainer as RefTrainer

    from torchtitan_b200.trainer import Trainer

    ref, ours = _config_tree(RefTrainer.Config), _config_tree(Trainer.Config)
    assert sorted(set(ref) - set(ours)) == []
    different = {k: (ref[k], ours[k]) for k in ref if not callable(ref[k]) and ref[k] != ours[k]}
    assert different == {}
    assert len(ref) > 100                                   # the walk really saw the whole tree


@pytest.mark.parametrize("family", ["llama3", "llama4", "qwen3", "deepseek_v3", "gpt_oss", "flux"])
def test_job_configurations_and_flavors_of_the_reference_exist(family):
    """Every job configuration function and every model flavor the reference registers for a family is registered here
    under the same name (``--module <family> --config <name>`` keeps working)."""
    import importlib
    import inspect

    if REF not in sys.path:
        sys.path.insert(0, REF)
    ref_reg = importlib.import_module(f"torchtitan.models.{family}.config_registry")
    our_reg = importlib.import_module(f"torchtitan_b200.models.{family}.config_registry")
    ref_jobs = {n for n, f in vars(ref_reg).items()
                if inspect.isfunction(f) and f.__module__ == ref_reg.__name__ and not n.startswith("_")}
    our_jobs = {n for n, f in vars(our_reg).items() if inspect.isfunction(f) and not n.startswith("_")}
    assert sorted(ref_jobs - our_jobs) == []
    ref_mod, our_mod = importlib.import_module(f"torchtitan.models.{family}"), importlib.import_module(f"torchtitan_b200.models.{family}")
    names = [a for a in dir(ref_mod) if a.endswith("_configs")]
    if names:
        ours = next(a for a in dir(our_mod) if a.endswith("_configs"))
        assert sorted(set(getattr(ref_mod, names[0])) - set(getattr(our_mod, ours))) == []


def test_flux_debug_flavor_matches_the_reference_model():
    """``flux-debug`` has the reference's dimensions (same parameter names and shapes) and, with the same weights, gives
    the same velocity field as the reference's FLUX model (fp32, CPU)."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.models.flux import flux_configs as ref_configs

    from torchtitan_b200.models.flux import flux_configs

    cfg = flux_configs["flux-debug"]
    torch.manual_seed(0)
    ours = cfg.build()
    ours.init_weights()
    torch.nn.init.normal_(ours.final_layer.linear.weight, std=0.02)      # the zero-initialised last layer would hide everything
    ref = ref_configs["flux-debug"].build()
    state = ours.state_dict()
    assert set(state) == set(ref.state_dict()) and all(v.shape == ref.state_dict()[k].shape for k, v in state.items())
    ref.load_state_dict(state)
    B, L, T = 2, 16, 8
    ids = torch.zeros(B, L, 3)
    ids[..., 1], ids[..., 2] = torch.arange(L).view(1, L) // 4, torch.arange(L).view(1, L) % 4
    kw = dict(img=torch.randn(B, L, 64), img_ids=ids, txt=torch.randn(B, T, cfg.context_in_dim), txt_ids=torch.zeros(B, T, 3),
              timesteps=torch.rand(B), y=torch.randn(B, cfg.vec_in_dim))
    with torch.no_grad():
        a, b = ours(**kw), ref(**kw)
    assert b.abs().max() > 0.1 and (a - b).abs().max().item() <= 1e-5 * b.abs().max().item()


@pytest.mark.parametrize("family", ["llama3", "llama4", "qwen3", "deepseek_v3", "gpt_oss", "flux"])
def test_every_flavor_has_the_reference_parameters(family):
    """Built on the meta device, every flavor of a family (debug models up to Llama-3.1-405B, DeepSeek-V3 671B, Qwen3
    235B-A22B, GPT-OSS 120b, FLUX dev) has exactly the parameter and buffer names and shapes of the reference's model, so
    checkpoints of either framework fit the other."""
    import importlib

    if REF not in sys.path:
        sys.path.insert(0, REF)

    def configs(mod):
        return getattr(mod, next(a for a in dir(mod) if a.endswith("_configs")))

    ours = configs(importlib.import_module(f"torchtitan_b200.models.{family}"))
    ref = configs(importlib.import_module(f"torchtitan.models.{family}"))
    for flavor in ref:
        with torch.device("meta"):
            a, b = ours[flavor].build().state_dict(), ref[flavor].build().state_dict()
        assert set(a) == set(b), (family, flavor, sorted(set(a) ^ set(b))[:4])
        wrong = [(k, tuple(a[k].shape), tuple(b[k].shape)) for k in a if a[k].shape != b[k].shape]
        assert not wrong, (family, flavor, wrong[:3])


def test_tokenizer_and_text_dataloader_give_the_reference_batches():
    """Same token ids as the reference's tokenizer wrapper (begin / end tokens, unicode, empty text) and, on the checked-in
    C4 sample, the same packed batches per data-parallel rank and the same loader state keys."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.components.tokenizer import HuggingFaceTokenizer as RefTokenizer
    from torchtitan.hf_datasets.text_datasets import HuggingFaceTextDataLoader as RefLoader

    from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer
    from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader

    assets = os.path.join(_HERE, "assets")
    ours_tok = HuggingFaceTokenizer(tokenizer_path=os.path.join(assets, "tokenizer"))
    ref_tok = RefTokenizer(tokenizer_path=os.path.join(assets, "tokenizer"))
    assert (ours_tok.get_vocab_size(), ours_tok.bos_id, ours_tok.eos_id) == (ref_tok.get_vocab_size(), ref_tok.bos_id, ref_tok.eos_id)
    for text in ["Hello world! 123", "  leading spaces\nand a newline\ttab", "ünïcödé 你好 🙂", ""]:
        for kw in (dict(add_bos=True, add_eos=True), dict(add_bos=False, add_eos=False), dict(add_bos=True, add_eos=False)):
            assert ours_tok.encode(text, **kw) == ref_tok.encode(text, **kw), (text, kw)
        assert ours_tok.decode(ours_tok.encode(text)) == ref_tok.decode(ref_tok.encode(text))
    data = os.path.join(assets, "c4_test")
    for world in (1, 2):
        for rank in range(world):
            kw = dict(dp_world_size=world, dp_rank=rank, seq_len=128, local_batch_size=2)
            ours = HuggingFaceTextDataLoader(HuggingFaceTextDataLoader.Config(dataset="c4_test", dataset_path=data), tokenizer=ours_tok, **kw)
            ref = RefLoader(RefLoader.Config(dataset="c4_test", dataset_path=data), tokenizer=ref_tok, **kw)
            a, b = iter(ours), iter(ref)
            for _ in range(6):
                (xa, ya), (xb, yb) = next(a), next(b)
                assert torch.equal(xa["input"], xb["input"]) and torch.equal(ya, yb), (world, rank)
            assert sorted(ours.state_dict()) == sorted(ref.state_dict())


def test_pipeline_stage_layouts_match_the_reference():
    """Automatic stage layouts (which layers, embedding and output go to which stage) for 1 - 8 stages, 1 - 39 layers and
    input / output weights 0 - 2: the same lists as the reference's function, and an error exactly where it raises."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torchtitan.distributed.pipeline_parallel import generate_llm_fqn_per_model_part as ref_layout

    from torchtitan_b200.parallel.pp import generate_llm_fqn_per_model_part as our_layout

    def run(fn, *a):
        try:
            return fn(*a)
        except ValueError:
            return "error"

    for stages in range(1, 9):
        for layers in range(1, 40):
            for in_w in (0, 1, 2):
                for out_w in (0, 1, 2):
                    case = (stages, layers, in_w, out_w)
                    assert run(our_layout, *case) == run(ref_layout, *case), case


@pytest.mark.parametrize("family", ["llama3", "llama4", "qwen3", "deepseek_v3", "gpt_oss"])
def test_parameter_and_flop_counts_match_the_reference(family):
    """The numbers behind the MFU / TFLOPs log line (parameters, FLOPs per token at sequence length 4096) equal the
    reference's for every flavor: dense, tied-embedding and mixture-of-experts (active parameters) formulas."""
    import importlib

    if REF not in sys.path:
        sys.path.insert(0, REF)

    def configs(mod):
        return getattr(mod, next(a for a in dir(mod) if a.endswith("_configs")))

    ours = configs(importlib.import_module(f"torchtitan_b200.models.{family}"))
    ref = configs(importlib.import_module(f"torchtitan.models.{family}"))
    for flavor in ref:
        with torch.device("meta"):
            a, b = ours[flavor].build(), ref[flavor].build()
        na, fa = ours[flavor].get_nparams_and_flops(a, 4096)
        nb, fb = ref[flavor].get_nparams_and_flops(b, 4096)
        assert na == nb and abs(fa - fb) <= 1e-9 * fb, (family, flavor, (na, fa), (nb, fb))


def test_grpo_loss_matches_the_reference_loss():
    """The GRPO objective (clipped ratio of per-sequence mean log-ratios, per-token KL estimate, entropy bonus) computed
    over one packed forward pass equals the reference's, which runs one forward pass per sequence: loss, metrics,
    per-token log-probabilities and parameter gradients; the log-probability identity report agrees as well."""
    import importlib.util

    # the file needs torch only; its package imports vLLM internals that this environment's vLLM does not have
    path = os.path.join(REF, "torchtitan", "experiments", "rl", "unified", "actors", "utils.py")
    if not os.path.exists(path):
        pytest.skip("the reference install has no rl/unified/actors/utils.py")
    spec = importlib.util.spec_from_file_location("_ref_rl_actor_utils", path)
    ref_utils = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_utils)

    from torchtitan_b200.experiments.rl import losses
    from torchtitan_b200.models.llama3 import llama3_configs

    cfg = dataclasses.replace(llama3_configs["debugmodel"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    torch.manual_seed(3)
    model = cfg.build()
    model.init_weights()
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 9, 3, 7)]
    gens = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 2, 11, 4)]
    adv = torch.tensor([0.7, -1.2, 0.1, 2.0])
    ref_lps = [torch.randn(len(x), generator=g) * 0.05 - 7.6 for x in gens]
    kw = dict(kl_coef=0.1, ppo_clip_eps=0.2, entropy_coef=0.01)

    want, want_metrics, want_lps = ref_utils.compute_policy_gradient_loss(model, gens, prompts, adv, ref_lps, **kw)
    want.backward()
    want_grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    got, got_metrics, got_lps = losses.compute_policy_gradient_loss(model, gens, prompts, adv, ref_lps, **kw)
    got.backward()
    assert got.item() == pytest.approx(want.item(), rel=1e-5)
    assert set(got_metrics) == set(want_metrics)
    for k in want_metrics:
        assert got_metrics[k] == pytest.approx(want_metrics[k], rel=1e-4, abs=1e-6), k
    for a, b in zip(got_lps, want_lps):
        assert torch.allclose(a, b, atol=1e-5)
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, want_grads[n], atol=1e-6 + 1e-4 * want_grads[n].abs().max().item()), n
    # micro-batches with the step's totals add up to the full-batch loss
    parts = [losses.compute_policy_gradient_loss(model, gens[i : i + 2], prompts[i : i + 2], adv[i : i + 2], ref_lps[i : i + 2],
                                                 n_seqs_total=4, n_tokens_total=sum(map(len, gens)), **kw)[0] for i in (0, 2)]
    assert (parts[0] + parts[1]).item() == pytest.approx(want.item(), rel=1e-5)
    fake_gen = [[float(v) for v in t.detach()] for t in got_lps]
    fake_gen[1][0] += 0.5
    assert losses.verify_logprob_identity(fake_gen, got_lps) == pytest.approx(ref_utils.verify_logprob_identity(fake_gen, got_lps))


def test_sum_digits_task_matches_the_reference_task():
    """Same questions for the same seed, same answer protocol in the system prompt, same answer extraction and rewards on completions of every
    kind the reward function distinguishes (tagged, prose, bare number, several tags, trailing text, wrong, empty)."""
    import importlib.util

    path = os.path.join(REF, "torchtitan", "experiments", "rl", "unified", "sum_digits.py")
    if not os.path.exists(path):
        pytest.skip("the reference install has no rl/unified/sum_digits.py")
    spec = importlib.util.spec_from_file_location("_ref_sum_digits", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    from torchtitan_b200.experiments.rl import sum_digits as ours

    a, b = ours.SumDigitsTask(seed=42), ref.SumDigitsTask(seed=42)
    assert [a.create_question() for _ in range(50)] == [b.create_question() for _ in range(50)]
    assert "[ANSWER] <number>" in a.get_system_prompt() and "[ANSWER] 28" in a.get_system_prompt()   # own wording, same protocol
    texts = ["[ANSWER] 28", "so the sum is 28", "the answer is 28.", "Answer: 27 [ANSWER] 28", "[ANSWER] 27 [ANSWER] 28",
             "[ANSWER] 28 and that is final", "1 + 2 = 28", "= 28. The answer", "[ANSWER] -28", "nothing here", "",
             "[ANSWER]   28  \n", "[ANSWER] 28\n[ANSWER] 28"]
    assert [ours.extract_answer(t) for t in texts] == [ref.extract_answer(t) for t in texts]
    for expected in ("28", "27", ""):
        assert torch.equal(a.reward_function(texts, expected), b.reward_function(texts, expected))


def test_vlm_model_matches_the_reference_model(monkeypatch):
    """Llama 3 + SigLIP-2 vision-language model: same parameter names, and with the same weights the same logits and
    gradients as the reference's model for a batch of two images of different grids scattered into two token rows (the
    reference's compiled flex attention replaced by the definition of attention under its own mask functions)."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from torch.nn.attention.flex_attention import create_block_mask

    import torchtitan.models.common.attention as ref_attention

    monkeypatch.setattr(ref_attention.FlexAttentionWrapper, "_compiled_flex_attn", staticmethod(_dense_flex_attention))
    monkeypatch.setattr(ref_attention, "_compiled_create_block_mask",
                        lambda *a, **k: create_block_mask(*a, **{**k, "device": "cpu"}))
    from torchtitan.experiments.vlm import llama3_siglip2_configs as ref_cfgs
    from torchtitan.experiments.vlm.model.args import SpecialTokens as RefSpecialTokens

    from torchtitan_b200.experiments.vlm import SpecialTokens, llama3_siglip2_configs as our_cfgs

    torch.manual_seed(0)
    cfg = our_cfgs["debugmodel"]
    ours = cfg.build()
    ours.init_weights()
    ref = ref_cfgs["debugmodel"].build()
    assert {k: v.shape for k, v in ours.state_dict().items()} == {k: v.shape for k, v in ref.state_dict().items()}
    with torch.no_grad():
        ref.init_weights(buffer_device=torch.device("cpu"))
    ref.load_state_dict(ours.state_dict())
    V, patch = cfg.vocab_size, cfg.encoder.patch_size
    img, boi, eoi, pad = V - 1, V - 2, V - 3, V - 4
    st = dict(img_token="<|image|>", img_id=img, boi_token="<|begin_of_image|>", boi_id=boi, eoi_token="<|end_of_image|>",
              eoi_id=eoi, pad_token="<|pad|>", pad_id=pad)
    B, S, N, L = 2, 96, 2, 16
    pixel = torch.zeros(N, L, 3 * patch * patch)
    grid = torch.full((N, L, 3), -1, dtype=torch.long)
    for n, (h, w) in enumerate([(3, 4), (2, 5)]):                     # 12 and 10 patches, padded to 16
        pixel[n, : h * w] = torch.randn(h * w, 3 * patch * patch)
        grid[n, : h * w] = torch.tensor([[0, i, j] for i in range(h) for j in range(w)])
    tokens = torch.randint(8, V - 8, (B, S))
    tokens[0, 5], tokens[0, 6:18], tokens[0, 18] = boi, img, eoi
    tokens[1, 30], tokens[1, 31:41], tokens[1, 41] = boi, img, eoi

    class _Tok:
        eos_id = 3

    tokens[0, 50] = _Tok.eos_id                                        # two documents in row 0
    lo = ours(tokens, pixel, grid, SpecialTokens(**st), attention_masks=ours.get_attention_masks(tokens, _Tok(), {"grid_thw": grid}))
    # the reference leaves the positional embeddings of padding patches uninitialised (torch.empty); whatever is there
    # reaches no real patch on a GPU kernel that skips masked keys, but 0 x NaN in the dense stand-in would: zero them
    with monkeypatch.context() as m:
        m.setattr(torch, "empty", torch.zeros)
        lr = ref(tokens, pixel, grid, RefSpecialTokens(**st), attention_masks=ref.get_attention_masks(tokens, _Tok(), {"grid_thw": grid}))
    assert (lo - lr).abs().max().item() < 2e-5 * max(lr.abs().max().item(), 1.0)
    lab = torch.randint(0, V, (B, S))
    torch.nn.functional.cross_entropy(lo.flatten(0, 1), lab.flatten()).backward()
    torch.nn.functional.cross_entropy(lr.flatten(0, 1), lab.flatten()).backward()
    ref_grads = dict(ref.named_parameters())
    for name, p in ours.named_parameters():
        g, w = p.grad, ref_grads[name].grad
        assert (g is None) == (w is None), name
        if g is not None:
            assert (g - w).abs().max().item() <= 1e-4 * max(w.abs().max().item(), 1e-6) + 1e-7, name


def _resolved(cfg, prefix="", out=None):
    """Flat ``{dotted option: value}`` of a job configuration object (the model specification left out)."""
    out = {} if out is None else out
    for f in dataclasses.fields(cfg):
        if f.name == "model_spec":
            continue
        v = getattr(cfg, f.name, None)
        if dataclasses.is_dataclass(v) and not isinstance(v, type):
            _resolved(v, prefix + f.name + ".", out)
        elif isinstance(v, list) and v and dataclasses.is_dataclass(v[0]):
            for i, x in enumerate(v):
                _resolved(x, f"{prefix}{f.name}.{i}.", out)
        else:
            out[prefix + f.name] = v
    return out


# options that deliberately resolve to other values than the reference's
_OWN_VALUES = {
    # files live elsewhere in this tree; the validation loader gets the job's encoder section and the shipped shard
    "models.flux": {"inference.prompts_path", "validator.dataloader.encoder.autoencoder_path", "validator.dataloader.encoder.t5_encoder",
                    "validator.dataloader.encoder.max_t5_encoding_len", "validator.dataloader.dataset"},
    # each job names its plan passes (the reference expects them on the command line) and keeps activation checkpointing
    "experiments.graph_trainer.llama3": {"compile.passes", "compile.joint_passes"},
    "experiments.graph_trainer.deepseek_v3": {"compile.passes", "compile.joint_passes", "activation_checkpoint.mode",
                                              "activation_checkpoint.selective_ac_option"},
}


@pytest.mark.parametrize("package", ["models.llama3", "models.llama4", "models.qwen3", "models.deepseek_v3", "models.gpt_oss",
                                     "models.flux", "experiments.vlm", "experiments.ft.llama3", "experiments.graph_trainer.llama3",
                                     "experiments.graph_trainer.deepseek_v3"])
def test_job_configurations_resolve_to_the_reference_values(package):
    """Every job configuration function of the reference exists here and resolves, option by option, to the same values
    (batch sizes, step counts, learning rates, schedules, checkpoint intervals, parallel degrees, checkpointing modes,
    datasets ...), apart from a short list of deliberate differences."""
    import importlib

    if REF not in sys.path:
        sys.path.insert(0, REF)
    ref = importlib.import_module(f"torchtitan.{package}.config_registry")
    ours = importlib.import_module(f"torchtitan_b200.{package}.config_registry")
    names = sorted(n for n in dir(ref) if not n.startswith("_") and n[0].islower() and callable(getattr(ref, n))
                   and getattr(getattr(ref, n), "__module__", "") == ref.__name__)
    assert names
    own = _OWN_VALUES.get(package, set())
    for name in names:
        assert hasattr(ours, name), f"{package}: job configuration {name} is missing"
        a, b = _resolved(getattr(ref, name)()), _resolved(getattr(ours, name)())
        assert sorted(set(a) - set(b)) == [], (name, sorted(set(a) - set(b)))
        different = {k: (a[k], b[k]) for k in a if not callable(a[k]) and a[k] != b[k] and k not in own}
        assert different == {}, (name, different)

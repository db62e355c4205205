"""Component logic that needs neither a GPU nor a process group: config manager, parallel-dims arithmetic, learning-rate
schedule, losses (model: the reference's CPU unit tests, tests/unit_tests/test_job_config.py, test_lr_scheduler.py,
test_parallel_dims.py)."""

import math

import pytest
import torch


# ------------------------------------------------------------------------------------------ config manager
def test_config_manager_loads_registry_function_and_applies_overrides():
    from torchtitan_b200.config.manager import ConfigManager

    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel",
        "--training.steps", "7", "--training.local_batch_size=3", "--parallelism.tensor_parallel_degree", "2",
        "--activation_checkpoint.mode", "full", "--optimizer.lr", "1e-3",
    ])
    assert cfg.training.steps == 7 and cfg.training.local_batch_size == 3
    assert cfg.parallelism.tensor_parallel_degree == 2
    assert cfg.activation_checkpoint.mode == "full"
    assert cfg.optimizer.lr == pytest.approx(1e-3)
    # untouched values keep what the registry function set
    base = ConfigManager().parse_args(["--module", "llama3", "--config", "llama3_debugmodel"])
    assert cfg.training.seq_len == base.training.seq_len


def test_config_manager_comma_separated_lists_and_errors():
    from torchtitan_b200.config.manager import ConfigManager

    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel",
        "--activation_checkpoint.per_op_sac_force_recompute_mm_shapes_by_fqns", "moe.router.gate,attention.wq",
    ])
    assert cfg.activation_checkpoint.per_op_sac_force_recompute_mm_shapes_by_fqns == ["moe.router.gate", "attention.wq"]
    with pytest.raises(ValueError, match="--module is required"):
        ConfigManager().parse_args(["--config", "llama3_debugmodel"])
    with pytest.raises(ValueError, match="--config is required"):
        ConfigManager().parse_args(["--module", "llama3"])
    with pytest.raises(ValueError, match="not found"):
        ConfigManager().parse_args(["--module", "llama3", "--config", "no_such_config"])
    with pytest.raises(ImportError):
        ConfigManager().parse_args(["--module", "no_such_model_family", "--config", "x"])
    with pytest.raises(SystemExit):      # unknown flag: the CLI parser rejects it
        ConfigManager().parse_args(["--module", "llama3", "--config", "llama3_debugmodel", "--training.no_such_key", "1"])


def test_config_manager_accepts_module_paths_and_every_registered_family():
    from torchtitan_b200.config.manager import ConfigManager
    from torchtitan_b200.models import _supported_models

    cfg = ConfigManager().parse_args(["--module", "torchtitan_b200.models.llama3", "--config", "llama3_debugmodel"])
    assert cfg.model_spec is not None
    for family in sorted(_supported_models):
        import importlib

        reg = importlib.import_module(f"torchtitan_b200.models.{family}.config_registry")
        names = [n for n in dir(reg) if "debug" in n and callable(getattr(reg, n)) and not n.startswith("_")]
        assert names, f"{family} has no debug config"
        c = ConfigManager().parse_args(["--module", family, "--config", names[0]])
        assert c.training.steps > 0


def test_parallelism_config_rejects_empty_load_balancer():
    from torchtitan_b200.config import ParallelismConfig

    with pytest.raises(ValueError):
        ParallelismConfig(context_parallel_load_balancer="")


# ------------------------------------------------------------------------------------------ parallel dims
def _pd(**kw):
    from torchtitan_b200.parallel import ParallelDims

    base = dict(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=1)
    base.update(kw)
    return ParallelDims(**base)


def test_parallel_dims_validation_and_leftover_shard_degree():
    pd = _pd(dp_shard=-1, tp=2, pp=2, world_size=16)
    assert pd.dp_shard == 4
    assert pd.dp_enabled and pd.fsdp_enabled and pd.tp_enabled and pd.pp_enabled and not pd.cp_enabled
    assert pd.non_data_parallel_size == 4
    with pytest.raises(AssertionError):
        _pd(dp_shard=3, tp=2, world_size=8)
    with pytest.raises(AssertionError):
        _pd(dp_shard=0, world_size=1)
    with pytest.raises(AssertionError):
        _pd(tp=0, world_size=1)
    with pytest.raises(AssertionError):            # ep * etp must divide dp_shard * cp * tp
        _pd(dp_shard=2, tp=2, ep=3, world_size=4)
    with pytest.raises(AssertionError):            # etp is 1 or tp
        _pd(dp_shard=2, tp=4, ep=2, etp=2, world_size=8)


def test_parallel_dims_rank_grids_follow_the_three_unflattenings():
    pd = _pd(dp_replicate=2, dp_shard=2, cp=2, tp=2, pp=2, ep=4, world_size=32)
    g = pd.grids
    assert g["dataloading"].sizes == (2, 4, 2, 2) and g["dataloading"].names == ("pp", "batch", "cp", "tp")
    assert g["dense"].sizes == (2, 2, 4, 2)         # fsdp = dp_shard * cp
    assert g["sparse"].sizes == (2, 2, 2, 4, 1)     # efsdp = fsdp * tp / (ep * etp)
    # tp is the fastest-varying dimension: ranks 0 and 1 share every coordinate but tp
    assert pd.ranks_of("tp", 0) == [0, 1]
    assert pd.coordinate("pp", 31) == 1 and pd.coordinate("pp", 0) == 0
    # an ep group of the sparse grid has ep members and they differ only in the ep coordinate
    ep_ranks = pd.ranks_of("ep", 5)
    assert len(ep_ranks) == 4 and 5 in ep_ranks
    assert pd.seq_len_divisor == 2 * 2 * 2         # tp * 2 * cp (head-tail halves)


def test_parallel_dims_gradient_divide_factor():
    pd = _pd(dp_replicate=2, dp_shard=4, cp=2, world_size=16)
    assert pd.fsdp_gradient_divide_factor == 2 * 4 * 2


# ------------------------------------------------------------------------------------------ learning-rate schedule
def _lrs(total, **kw):
    from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer

    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    sched = LRSchedulersContainer(LRSchedulersContainer.Config(**kw), optimizers=[opt], training_steps=total)
    out = []
    for _ in range(total):
        out.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    return out, sched, opt


def test_lr_warmup_then_linear_decay_to_zero():
    lrs, _, _ = _lrs(10, warmup_steps=2, decay_type="linear")
    assert lrs[0] == pytest.approx(1 / 2) and lrs[1] == pytest.approx(1.0)   # the last warm-up step is at the peak
    assert lrs[2] == pytest.approx(1.0)                       # one stable step (the virtual extra step)
    assert all(a > b for a, b in zip(lrs[2:], lrs[3:]))       # then strictly decreasing
    assert lrs[3] == pytest.approx(1 - 1 / 8)
    assert lrs[-1] == pytest.approx(1 - 7 / 8) and lrs[-1] > 0.0


def test_lr_warmup_stable_decay_with_floor_and_shapes():
    lrs, _, _ = _lrs(20, warmup_steps=2, decay_ratio=0.25, decay_type="cosine", min_lr_factor=0.1)
    assert lrs[2:15] == pytest.approx([1.0] * 13)               # plateau until the last quarter
    assert min(lrs[15:]) >= 0.1 - 1e-9
    lin, _, _ = _lrs(20, warmup_steps=2, decay_ratio=0.25, decay_type="linear")
    sq, _, _ = _lrs(20, warmup_steps=2, decay_ratio=0.25, decay_type="sqrt")
    cos, _, _ = _lrs(20, warmup_steps=2, decay_ratio=0.25, decay_type="cosine")
    # one step into the decay: sqrt falls fastest, cosine slowest
    assert sq[17] < lin[17] < cos[17]


def test_lr_schedule_clamps_oversized_warmup_and_round_trips_state():
    lrs, sched, opt = _lrs(4, warmup_steps=10)
    assert lrs == sorted(lrs)                                    # still warming up at the end
    from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer

    state = sched.state_dict()
    opt2 = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s2 = LRSchedulersContainer(LRSchedulersContainer.Config(warmup_steps=10), optimizers=[opt2], training_steps=4)
    s2.load_state_dict(state)
    assert s2.state_dict()["last_epoch"] == state["last_epoch"]
    with pytest.raises(AssertionError):
        LRSchedulersContainer(LRSchedulersContainer.Config(), optimizers=[], training_steps=4)


def test_wsd_multiplier_rejects_unknown_shape():
    from torchtitan_b200.components.lr_scheduler import wsd_multiplier

    with pytest.raises(ValueError):
        wsd_multiplier(5, warmup=1, stable=1, decay=5, kind="exp", floor=0.0)
    assert wsd_multiplier(0, warmup=0, stable=3, decay=2, kind="linear", floor=0.0) == 1.0


# ------------------------------------------------------------------------------------------ losses
def test_cross_entropy_is_a_token_sum_that_skips_ignored_labels():
    from torchtitan_b200.components.loss import IGNORE_INDEX, build_cross_entropy_loss, build_mse_loss

    torch.manual_seed(0)
    logits = torch.randn(2, 5, 11, requires_grad=True)
    labels = torch.randint(0, 11, (2, 5))
    labels[0, 1] = IGNORE_INDEX
    loss = build_cross_entropy_loss()(logits, labels)
    want = torch.nn.functional.cross_entropy(logits.flatten(0, 1).float(), labels.flatten(), reduction="sum", ignore_index=IGNORE_INDEX)
    assert loss.dtype == torch.float32 and torch.allclose(loss, want, atol=1e-5)
    loss.backward()
    assert logits.grad[0, 1].abs().sum() == 0          # the ignored token gets no gradient
    # bf16 logits are reduced in fp32
    lb = build_cross_entropy_loss()(logits.detach().bfloat16(), labels)
    assert lb.dtype == torch.float32 and math.isfinite(float(lb))
    mse = build_mse_loss()(torch.ones(3, 4), torch.zeros(3, 4))
    assert float(mse) == 12.0


def test_every_registered_job_configuration_parses(monkeypatch):
    """``--module <m> --config <c>`` goes through the command-line parser for every job configuration of every model
    family and experiment, including those whose converter list holds two converter kinds (both nested classes are
    called ``Config``, which the parser could not tell apart), and an option of the second converter can be overridden."""
    import importlib

    from torchtitan_b200.config.manager import ConfigManager
    from torchtitan_b200.experiments import _supported_experiments
    from torchtitan_b200.models import _supported_models

    monkeypatch.setenv("WORLD_SIZE", "8")           # the planner-driven configurations size themselves for the job
    seen = 0
    for kind, names in (("models", sorted(_supported_models)), ("experiments", sorted(_supported_experiments))):
        for m in names:
            try:
                reg = importlib.import_module(f"torchtitan_b200.{kind}.{m}.config_registry")
            except ModuleNotFoundError:
                continue                             # an experiment without job configurations of its own
            for c in sorted(n for n in dir(reg) if not n.startswith("_") and n[0].islower() and callable(getattr(reg, n))
                            and getattr(getattr(reg, n), "__module__", "") == reg.__name__):
                flat = m != "rl"                       # the RL job nests a trainer and a generator configuration
                cfg = ConfigManager().parse_args(["--module", m, "--config", c] + (["--training.steps", "3"] if flat else []))
                assert cfg is not None and (not flat or cfg.training.steps == 3), (m, c)
                seen += 1
    assert seen > 40
    cfg = ConfigManager().parse_args([
        "--module", "deepseek_v3", "--config", "deepseek_v3_671b",
        "model-converters.converters.1:float8-grouped-mm-converter-config", "--model-converters.converters.1.fqns", "abc"])
    kinds = [type(c).__qualname__ for c in cfg.model_converters.converters]
    assert kinds == ["Float8LinearConverter.Config", "Float8GroupedMMConverter.Config"]
    assert cfg.model_converters.converters[1].fqns == ["abc"]
    assert type(cfg.model_converters.converters[0]).__name__ == "Config"        # the temporary names are gone again

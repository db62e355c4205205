"""The training loop end to end on CPU: loss goes down, a run resumed from a checkpoint continues bit for bit, stale
checkpoints are purged, the last step can be exported model-only, and validation runs (model: the reference's integration
tests "checkpoint save / load / model-only last step" in tests/integration_tests/features.py and
tests/unit_tests/test_checkpoint.py)."""

import os

import pytest
import torch


def _trainer(tmp_path, steps, extra=(), config="llama3_debugmodel_synthetic"):
    from dist_utils import free_port
    from torchtitan_b200.config.manager import ConfigManager

    os.environ["MASTER_PORT"] = str(free_port())            # every (re)initialised process group gets its own rendezvous port

    args = [
        "--module", "llama3", "--config", config, "--dump_folder", str(tmp_path),
        "--training.steps", str(steps), "--training.local_batch_size", "2", "--training.seq_len", "64",
        "--training.dtype", "float32", "--metrics.log_freq", "1", "--lr_scheduler.warmup_steps", "2",
        "--debug.seed", "7", "--debug.deterministic",
    ] + (["--validator.freq", "1000"] if "synthetic" in config else [])
    flags, sets = [], {}
    extra = list(extra)
    while extra:                                             # "--a.b", "False"/"True" pairs are set on the parsed config
        k = extra.pop(0)
        if extra and extra[0] in ("True", "False"):
            sets[k.lstrip("-")] = extra.pop(0) == "True"
        else:
            flags.append(k)
    cfg = ConfigManager().parse_args(args + flags)
    for path, val in sets.items():
        obj = cfg
        *head, leaf = path.split(".")
        for h in head:
            obj = getattr(obj, h)
        setattr(obj, leaf, val)
    return cfg.build()


def _run(tr, n=None):
    """Step the trainer like ``train()`` does, recording the loss of every step."""
    it = tr.batch_generator(tr.dataloader)
    losses = []
    while tr.should_continue_training() and (n is None or len(losses) < n):
        tr.step += 1
        tr.train_step(it)
        tr.checkpointer.save(tr.step, last_step=(tr.step == tr.config.training.steps))
        losses.append(float(tr.last_loss))
    return losses


@pytest.fixture()
def single_rank(monkeypatch):
    import torch.distributed as dist

    if dist.is_initialized():          # an earlier in-process trainer test of this worker may have left its group behind
        dist.destroy_process_group()
    monkeypatch.setenv("LOCAL_RANK", "0")
    yield

    if dist.is_initialized():
        dist.destroy_process_group()


def test_debug_model_trains_on_text_and_loss_decreases(tmp_path, single_rank):
    """Tokenizer + packed text dataset (the checked-in c4 sample) + model + optimizer: real text is learnable."""
    tr = _trainer(tmp_path, 12, ["--training.local_batch_size", "4", "--training.seq_len", "128"], config="llama3_debugmodel")
    losses = _run(tr)
    tr.close()
    assert len(losses) == 12 and all(l == l for l in losses)
    assert sum(losses[-3:]) / 3 < sum(losses[:3]) / 3 - 0.3, losses


def test_resume_from_checkpoint_continues_bitwise(tmp_path, single_rank):
    import torch.distributed as dist

    ck = ["--checkpoint.enable", "--checkpoint.interval", "3", "--checkpoint.folder", "ckpt",
          "--checkpoint.last_save_model_only", "False"]
    full = _trainer(tmp_path / "a", 8, ck)
    want = _run(full)
    full.close()
    dist.destroy_process_group()

    first = _trainer(tmp_path / "b", 8, ck)
    got = _run(first, n=5)                                  # checkpoints at steps 3 (and 6 is never reached)
    first.close()
    dist.destroy_process_group()
    assert sorted(os.listdir(tmp_path / "b" / "ckpt")) == ["step-3"]

    resumed = _trainer(tmp_path / "b", 8, ck)
    assert resumed.checkpointer.load(step=-1)
    assert resumed.step == 3
    rest = _run(resumed)
    resumed.close()
    assert got[:3] == want[:3]
    assert rest == want[3:], (rest, want[3:])               # model, optimizer, schedule and data position all restored


def test_keep_latest_k_and_model_only_last_step(tmp_path, single_rank):
    ck = ["--checkpoint.enable", "--checkpoint.interval", "2", "--checkpoint.folder", "ckpt", "--checkpoint.keep_latest_k", "2",
          "--checkpoint.last_save_model_only", "True", "--checkpoint.export_dtype", "bfloat16"]
    tr = _trainer(tmp_path, 7, ck)
    _run(tr)
    tr.close()                                               # joins the purge thread
    kept = sorted(os.listdir(tmp_path / "ckpt"), key=lambda s: int(s.split("-")[1]))
    # interval saves keep the latest two (step-2 was purged when step-6 landed); the final export is written without a purge
    assert kept == ["step-4", "step-6", "step-7"], kept
    # the last step holds the model only, in the export dtype
    import torch.distributed.checkpoint as dcp

    meta = dcp.FileSystemReader(str(tmp_path / "ckpt" / "step-7")).read_metadata()
    keys = list(meta.state_dict_metadata)
    assert keys and not any(k.startswith(("optimizer", "lr_scheduler", "dataloader", "train_state")) for k in keys)
    assert all(m.properties.dtype == torch.bfloat16 for m in meta.state_dict_metadata.values() if hasattr(m, "properties"))
    full_keys = list(dcp.FileSystemReader(str(tmp_path / "ckpt" / "step-6")).read_metadata().state_dict_metadata)
    assert any(k.startswith("optimizer") for k in full_keys) and any(k.startswith("train_state") for k in full_keys)


def test_exclude_from_loading_and_missing_step(tmp_path, single_rank):
    import torch.distributed as dist

    ck = ["--checkpoint.enable", "--checkpoint.interval", "2", "--checkpoint.folder", "ckpt",
          "--checkpoint.last_save_model_only", "False"]
    tr = _trainer(tmp_path, 4, ck)
    _run(tr)
    w = tr.model_parts[0].output.weight.detach().clone()
    tr.close()
    dist.destroy_process_group()
    again = _trainer(tmp_path, 4, ck + ["--checkpoint.exclude_from_loading", "lr_scheduler,dataloader"])
    assert again.checkpointer.load(step=2)
    assert again.step == 2
    with pytest.raises(FileNotFoundError):
        again.checkpointer.load(step=3)
    assert again.checkpointer.load(step=4)
    assert torch.equal(again.model_parts[0].output.weight.detach(), w)
    again.close()


def test_validation_and_gradient_accumulation(tmp_path, single_rank):
    tr = _trainer(tmp_path, 2, ["--validator.enable", "True", "--validator.freq", "1", "--validator.steps", "2",
                                "--training.global_batch_size", "4"])
    assert tr.gradient_accumulation_steps == 2
    losses = _run(tr)
    assert tr.validator is not None and tr.validator.should_validate(1)
    tr.validator.validate(tr.model_parts, tr.step)
    tr.close()
    assert len(losses) == 2


def test_last_step_export_in_hf_format_and_reload(tmp_path, single_rank):
    """The final model-only checkpoint can be written as Hugging Face safetensors (names converted by the model's
    state-dict adapter) and a new run can start from it through ``initial_load_in_hf``."""
    import glob

    import torch.distributed as dist
    from safetensors import safe_open

    ck = ["--checkpoint.enable", "--checkpoint.interval", "100", "--checkpoint.folder", "ckpt",
          "--checkpoint.last_save_model_only", "True", "--checkpoint.last_save_in_hf", "True"]
    tr = _trainer(tmp_path, 2, ck)
    _run(tr)
    w = tr.model_parts[0].layers["0"].attention.wq.weight.detach().clone()
    out = tr.model_parts[0].output.weight.detach().clone()
    tr.close()
    dist.destroy_process_group()
    files = glob.glob(str(tmp_path / "ckpt" / "step-2" / "*.safetensors"))
    assert files
    names = set()
    for f in files:
        with safe_open(f, "pt") as sf:
            names |= set(sf.keys())
    assert "model.embed_tokens.weight" in names and "model.layers.0.self_attn.q_proj.weight" in names and "lm_head.weight" in names
    fresh = _trainer(tmp_path / "second", 2, ["--checkpoint.enable", "--checkpoint.folder", "ckpt2",
                                               "--checkpoint.initial_load_path", str(tmp_path / "ckpt" / "step-2"),
                                               "--checkpoint.initial_load_in_hf", "True"])
    assert fresh.checkpointer.load(step=-1)
    assert fresh.step == 0                                    # model only: the run starts from step 0 with these weights
    assert torch.equal(fresh.model_parts[0].output.weight.detach(), out)
    assert torch.allclose(fresh.model_parts[0].layers["0"].attention.wq.weight.detach(), w)
    fresh.close()


def test_no_checkpoint_is_written_after_a_kernel_gave_up(tmp_path, single_rank):
    """A kernel error word that shows up between log steps stops the run before the step's checkpoint is written (the
    interval is not a multiple of the log frequency, so only the check in front of the save can catch it)."""
    ck = ["--checkpoint.enable", "--checkpoint.interval", "3", "--checkpoint.folder", "ckpt", "--metrics.log_freq", "100"]
    tr = _trainer(tmp_path, 8, ck)
    seen = []

    def fake_words(sync=False):
        seen.append((tr.step, sync))
        return {"comm": 1} if tr.step >= 6 else {}

    tr._kernel_error_words = fake_words
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        tr.train()
    tr.close()
    assert sorted(os.listdir(tmp_path / "ckpt")) == ["step-3"]          # step-6 was never written
    assert (3, True) in seen and (6, True) in seen                       # checked (with a sync) right before both saves

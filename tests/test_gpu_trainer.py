"""The training loop on one GPU through the public config + trainer API: the CUDA kernels, the single-device mixed-precision
units and the flat-shard optimizer train the debug model on the checked-in text sample, a resumed run continues bit for bit,
and no kernel reports an expired wait."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(tmp_path, steps, extra=()):
    from dist_utils import free_port
    from torchtitan_b200.config.manager import ConfigManager

    os.environ["MASTER_PORT"] = str(free_port())
    os.environ.setdefault("LOCAL_RANK", "0")
    args = ["--module", "llama3", "--config", "llama3_debugmodel", "--dump_folder", str(tmp_path), "--training.steps", str(steps),
            "--training.local_batch_size", "4", "--training.seq_len", "512", "--metrics.log_freq", "1",
            "--lr_scheduler.warmup_steps", "2", "--debug.seed", "11"] + list(extra)
    return ConfigManager().parse_args(args).build()


def _run(tr, n=None):
    it = tr.batch_generator(tr.dataloader)
    losses = []
    while tr.should_continue_training() and (n is None or len(losses) < n):
        tr.step += 1
        tr.train_step(it)
        tr.checkpointer.save(tr.step, last_step=(tr.step == tr.config.training.steps))
        losses.append(float(tr.last_loss))
    return losses


def test_gpu_training_learns_and_uses_native_kernels(tmp_path):
    from torchtitan_b200.ops import native

    before = native.CALLS
    tr = _trainer(tmp_path, 12)
    assert tr.device.type == "cuda"
    losses = _run(tr)
    tr.close()
    torch.cuda.synchronize()
    assert all(l == l for l in losses) and sum(losses[-3:]) / 3 < sum(losses[:3]) / 3 - 0.3, losses
    assert native.CALLS - before > 12 * 50                # the hot ops went through the native library, not a fallback
    assert not native.kernel_errors()


def test_gpu_resume_is_bitwise(tmp_path):
    import torch.distributed as dist

    # deterministic algorithms: the debug model's head dimension (16) takes PyTorch's attention, whose default backward
    # adds dQ with atomics (and so does this framework's fused backward for head dimension 128)
    ck = ["--checkpoint.enable", "--checkpoint.interval", "3", "--checkpoint.folder", "ckpt", "--debug.deterministic",
          "--debug.deterministic_warn_only"]

    def build(path, steps):
        tr = _trainer(path, steps, ck)
        tr.config.checkpoint.last_save_model_only = False
        tr.checkpointer.last_save_model_only = False
        return tr

    full = build(tmp_path / "a", 6)
    want = _run(full)
    full.close()
    dist.destroy_process_group()
    first = build(tmp_path / "b", 6)
    got = _run(first, n=4)
    first.close()
    dist.destroy_process_group()
    resumed = build(tmp_path / "b", 6)
    assert resumed.checkpointer.load(step=-1) and resumed.step == 3
    rest = _run(resumed)
    resumed.close()
    assert got[:3] == want[:3] and rest == want[3:], (want, got, rest)

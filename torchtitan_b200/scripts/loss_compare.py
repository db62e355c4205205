"""Compare the loss curves of two training scenarios, optionally asserting bit-exact equality.

A scenario is (git commit or ``.`` for the working tree, module, config, extra options, number of GPUs). Both runs get
``--debug.deterministic --debug.seed=42 --metrics.enable_tensorboard --metrics.log_freq=1``, start from the same seed
checkpoint unless ``--no-seed-checkpoint`` is given, and their per-step ``loss_metrics/global_avg_loss`` values are
read back (TensorBoard event files when the reader is available, else the ``step: N  loss: X`` log lines).
``--assert-equal`` requires identical values at every step; ``--export-result`` / ``--import-result`` write / read the
loss table so that a run can be checked against a stored golden file.
Parity: scripts/loss_compare.py (options and defaults :899-1000, fixed options :72-82, comparison :703-834)."""

from __future__ import annotations

import argparse
import os
import re
import shlex
import shutil
import subprocess
import sys

LOG_PREFIX = "[LOSS_COMPARE]"
TB_LOSS_TAG = "loss_metrics/global_avg_loss"
FIXED_OPTIONS = "--debug.deterministic --debug.seed=42 --metrics.enable_tensorboard --metrics.log_freq=1"
_ANSI = re.compile(r"\x1b\[[0-9;]*m")
_STEP = re.compile(r"step:\s*(\d+)\s+loss:\s*(-?[0-9.]+(?:e[-+]?\d+)?)")


def log(msg: str) -> None:
    print(f"{LOG_PREFIX} {msg}", flush=True)


def build_command(module: str, config: str, ngpus: int, steps: int, options: str, dump_folder: str, seed_ckpt: str | None) -> list[str]:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ngpus}", "--master-addr", "127.0.0.1",
           "--master-port", os.environ.get("LOSS_COMPARE_PORT", "29533"), "-m", "torchtitan_b200.train",
           "--module", module, "--config", config, f"--training.steps={steps}", f"--dump_folder={dump_folder}"]
    cmd += shlex.split(FIXED_OPTIONS)
    if seed_ckpt:
        cmd += ["--checkpoint.enable", f"--checkpoint.initial_load_path={seed_ckpt}", "--checkpoint.initial_load_model_only",
                "--checkpoint.interval=1000000"]
    cmd += shlex.split(options)
    return cmd


def parse_losses_from_log(text: str) -> dict[int, float]:
    out: dict[int, float] = {}
    for line in text.splitlines():
        line = _ANSI.sub("", line)
        if "validate" in line:
            continue
        m = _STEP.search(line)
        if m:
            out[int(m.group(1))] = float(m.group(2))
    return out


def read_tensorboard_losses(folder: str) -> dict[int, float]:
    try:
        from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    except ImportError:
        return {}
    out: dict[int, float] = {}
    for root, _, files in os.walk(folder):
        if any(f.startswith("events.out.tfevents") for f in files):
            acc = EventAccumulator(root)
            acc.Reload()
            if TB_LOSS_TAG in acc.Tags().get("scalars", []):
                for ev in acc.Scalars(TB_LOSS_TAG):
                    out[ev.step] = ev.value
    return out


def checkout(commit: str, workdir: str) -> str:
    """Returns the source directory for ``commit`` (a detached worktree), or the current tree for ``.``."""
    if commit in (".", ""):
        return os.getcwd()
    dst = os.path.join(workdir, f"src_{commit[:12]}")
    if not os.path.exists(dst):
        subprocess.run(["git", "worktree", "add", "--detach", dst, commit], check=True)
    return dst


def run_scenario(name: str, commit: str, module: str, config: str, ngpus: int, steps: int, options: str, out_dir: str,
                 seed_ckpt: str | None) -> dict[int, float]:
    src = checkout(commit, out_dir)
    dump = os.path.join(out_dir, f"{name}_outputs")
    shutil.rmtree(dump, ignore_errors=True)
    cmd = build_command(module, config, ngpus, steps, options, dump, seed_ckpt)
    log(f"{name}: {' '.join(cmd)} (cwd={src})")
    r = subprocess.run(cmd, cwd=src, capture_output=True, text=True)
    with open(os.path.join(out_dir, f"{name}.log"), "w") as f:
        f.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"{name} run failed, see {out_dir}/{name}.log")
    losses = read_tensorboard_losses(dump) or parse_losses_from_log(r.stdout + r.stderr)
    if not losses:
        raise RuntimeError(f"no losses found for {name}")
    return losses


def create_seed_checkpoint(module: str, config: str, options: str, out_dir: str) -> str:
    dump = os.path.join(out_dir, "seed_outputs")
    shutil.rmtree(dump, ignore_errors=True)
    cmd = [sys.executable, "-m", "torchtitan_b200.train", "--module", module, "--config", config, f"--dump_folder={dump}",
           "--checkpoint.enable", "--checkpoint.create_seed_checkpoint", "--debug.seed=42", "--debug.deterministic",
           "--parallelism.data_parallel_shard_degree=1"] + shlex.split(options)
    env = dict(os.environ, WORLD_SIZE="1", RANK="0", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29534")
    subprocess.run(cmd, check=True, env=env, capture_output=True, text=True)
    return os.path.join(dump, "checkpoint", "step-0")


def export_losses(path: str, losses: dict[int, float]) -> None:
    with open(path, "w") as f:
        for s in sorted(losses):
            f.write(f"{s} {losses[s]!r}\n")


def import_losses(path: str) -> dict[int, float]:
    out = {}
    with open(path) as f:
        for line in f:
            if line.strip():
                s, v = line.split()
                out[int(s)] = float(v)
    return out


def compare(a: dict[int, float], b: dict[int, float], assert_equal: bool, names=("baseline", "test")) -> bool:
    steps = sorted(set(a) | set(b))
    log(f"{'step':>6} {names[0]:>14} {names[1]:>14} {'diff':>12}")
    equal = set(a) == set(b)
    for s in steps:
        va, vb = a.get(s), b.get(s)
        d = (vb - va) if (va is not None and vb is not None) else float("nan")
        log(f"{s:>6} {va if va is not None else float('nan'):>14.6f} {vb if vb is not None else float('nan'):>14.6f} {d:>12.3e}")
        equal = equal and va == vb
    if assert_equal and not equal:
        log("losses differ")
    return equal


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("baseline_commit", help="Git commit hash for baseline ('.' = working tree)")
    p.add_argument("test_commit", help="Git commit hash for test ('.' = working tree)")
    p.add_argument("--baseline-module", default="llama3")
    p.add_argument("--test-module", default="")
    p.add_argument("--baseline-config", default="llama3_debugmodel")
    p.add_argument("--test-config", default="")
    p.add_argument("--baseline-options", default="")
    p.add_argument("--test-options", default="")
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--no-seed-checkpoint", action="store_true")
    p.add_argument("--output-folder", default="")
    p.add_argument("--assert-equal", action="store_true")
    p.add_argument("--export-result", default="")
    p.add_argument("--import-result", default="")
    p.add_argument("--job-dump-folder", default="outputs")
    p.add_argument("--baseline-ngpus", type=int, default=8)
    p.add_argument("--test-ngpus", type=int, default=8)
    a = p.parse_args(argv)
    if a.export_result and not a.assert_equal:
        p.error("--export-result requires --assert-equal")
    out_dir = a.output_folder or os.path.join(a.job_dump_folder, "loss_compare")
    os.makedirs(out_dir, exist_ok=True)
    test_module, test_config = a.test_module or a.baseline_module, a.test_config or a.baseline_config
    seed = None if a.no_seed_checkpoint else create_seed_checkpoint(a.baseline_module, a.baseline_config, a.baseline_options, out_dir)
    test = run_scenario("test", a.test_commit, test_module, test_config, a.test_ngpus, a.steps, a.test_options, out_dir, seed)
    if a.import_result:
        base, names = import_losses(a.import_result), ("imported", "test")
    else:
        base = run_scenario("baseline", a.baseline_commit, a.baseline_module, a.baseline_config, a.baseline_ngpus, a.steps,
                            a.baseline_options, out_dir, seed)
        names = ("baseline", "test")
    equal = compare(base, test, a.assert_equal, names)
    if a.export_result and equal:
        export_losses(a.export_result, test)
    if a.assert_equal and not equal:
        return 1
    log("done")
    return 0


if __name__ == "__main__":
    sys.exit(main())

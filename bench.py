"""Headline benchmark: Llama-3.1-8B pre-training throughput (tokens/s, whole job) on N B200s.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Config (same as the reference's ``llama3_8b``): dim 4096, 32 layers, 32/8 heads, FFN 14336, vocab
128256, local batch 1 x seq 8192 per GPU, FSDP over all GPUs, bf16 compute with fp32 master
weights and fp32 gradient reduction, selective (per-op) activation checkpointing, AdamW with
gradient clipping; synthetic uniform tokens from seed 0 and random-init weights.

Two timed regions of K optimizer steps each (after W warm-up steps), both bracketed by a barrier
and ``torch.cuda.synchronize()`` and timed with CUDA events, max over ranks:
  * ``value``: batches already resident on the device (the kernel/collective time of a step);
  * ``e2e``: the public ``Trainer.train_step`` path fed by the data loader's pinned host batches
    (host->device copy every step) plus a device->host read of the loss every step.
``--impl reference`` runs the unmodified reference installed under ``baseline/_ref`` on the same
config, eager and with its own ``--compile.enable``, and prints the faster build's JSON line with
``"impl": "reference"`` (``config.compile`` says which). Both arms use the same selective-checkpoint
policy (every second matmul output kept); ``--sac-mm-policy auto`` keeps all of them when memory allows.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_TOK_S_PER_GPU = 8307.5  # reference docs/mxfp8.md:152, 8xB200 bf16 FSDP2 + compile
SEQ_LEN = 8192
MODEL = "llama3_8b"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # idle samples (before the first kernel) would drag the median down: keep the upper half
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def build_trainer(n_gpus: int, steps_total: int, ac_mode: str | None = None, layers: int | None = None,
                  extra: list[str] | None = None, sac_mm_policy: str = "every_second", config: str = "llama3_8b_synthetic"):
    from torchtitan_b200.config.manager import ConfigManager
    from torchtitan_b200.models.llama3 import llama3_configs

    if layers is not None:  # profiling aid only: a truncated model is not a benchmark result
        llama3_configs["8B"].n_layers = layers

    args = [
        "--module", "llama3", "--config", config,
        "--training.steps", str(steps_total), "--metrics.log_freq", "1000000",
        "--dump_folder", "/tmp/tt_b200_bench", "--comm.train_timeout_seconds", "300",
        # which matmul outputs per-op SAC keeps: "every_second" is the reference's policy (both arms then recompute the
        # same share of the forward); "all" / "auto" trade memory for less recompute and are labelled in the output
        "--activation_checkpoint.per_op_sac_mm_policy", sac_mm_policy,
    ]
    if ac_mode:
        args += ["--activation_checkpoint.mode", ac_mode]
    args += list(extra or [])
    cfg = ConfigManager().parse_args(args)
    return cfg.build()


def _sac_mm_policy(trainer) -> str:
    from torchtitan_b200.parallel import ac

    mode = trainer.config.activation_checkpoint.per_op_sac_mm_policy
    if mode == "auto":
        return "all (auto: memory allows)" if ac._AUTO_KEEP_ALL else "every second (auto: memory bound)"
    return mode


def max_over_ranks(x: float) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync():
    import torch
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier(device_ids=[torch.cuda.current_device()])
    torch.cuda.synchronize()


def write_kernel_table(path: str, step_fn, rank: int) -> None:
    """Run one more step under the PyTorch profiler (device activities only) and write the time per kernel name,
    largest first, as text. The figures are in-situ durations (clocks and caches as in training); they are a
    breakdown, not a benchmark value."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn()
        torch.cuda.synchronize()
    if rank != 0:
        return
    rows: dict[str, list[float]] = {}
    for ev in prof.events():
        if ev.device_type is not None and str(ev.device_type).endswith("CUDA"):
            r = rows.setdefault(ev.name, [0.0, 0])
            r[0] += ev.device_time_total if hasattr(ev, "device_time_total") else ev.cuda_time_total
            r[1] += 1
    total = sum(v[0] for v in rows.values()) or 1.0
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(f"# device time of one step by kernel (us); total {total:.0f} us\n")
        for name, (us, n) in sorted(rows.items(), key=lambda kv: -kv[1][0])[:60]:
            f.write(f"{us:12.0f} {100 * us / total:6.2f}% {n:6d}  {name[:150]}\n")


def run_ours(args) -> dict:
    import torch

    from torchtitan_b200.ops import native
    from torchtitan_b200.tools.logging import init_logger

    rank, world, local = _dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    if rank == 0:
        init_logger()
    total_steps = args.warmup + 2 * args.steps + 4
    trainer = build_trainer(args.gpus, total_steps, args.ac, args.layers, args.override, args.sac_mm_policy, args.config)
    dev = trainer.device
    local_bs = trainer.config.training.local_batch_size
    pd = trainer.parallel_dims
    # a step consumes local_bs sequences per rank of the batch (data-parallel) mesh; ranks of a tensor / context /
    # pipeline group work on the same sequences
    batch_degree = pd.dp_replicate * pd.dp_shard
    tokens_per_step = local_bs * SEQ_LEN * batch_degree
    dims = [("dp_replicate", pd.dp_replicate), ("fsdp", pd.dp_shard), ("cp", pd.cp), ("tp", pd.tp), ("pp", pd.pp), ("ep", pd.ep)]
    parallelism = "x".join(f"{n}{d}" for n, d in dims if d > 1) or "single-gpu (fp32 master + bf16 compute copy)"

    host_iter = trainer.batch_generator(trainer.dataloader)

    def device_iter():
        # batches staged on the device ahead of the timed region (distinct data every step)
        staged = []
        for _ in range(args.steps):
            d, l = next(host_iter)
            staged.append(({k: v.to(dev) for k, v in d.items()}, l.to(dev)))
        torch.cuda.synchronize()
        for item in staged:
            yield item

    def step(it):
        trainer.step += 1
        trainer.train_step(it)

    for _ in range(args.warmup):
        step(host_iter)
    barrier_sync()
    assert not native.kernel_errors(), "kernel error flag set during warm-up"

    # ---- region 1: device-resident inputs ------------------------------------------------
    dit = device_iter()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    calls0 = native.CALLS
    barrier_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(dit)
    e1.record()
    barrier_sync()
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = native.CALLS - calls0
    clocks = sampler.stop() if rank == 0 else {}

    # ---- region 2: end to end (pinned host batch -> device every step, loss read back) ---------
    h2d = 0
    barrier_sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last_loss = None
    for _ in range(args.steps):
        step(host_iter)
        last_loss = float(trainer.last_loss.item())  # 4-byte device->host read, syncs the step
    f1.record()
    barrier_sync()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1)) / args.steps
    h2d = 2 * local_bs * SEQ_LEN * 8  # int64 inputs + labels per rank per step
    errs = native.kernel_errors()
    mem_gib = torch.cuda.max_memory_reserved() / 2**30
    value = tokens_per_step / (dev_ms / 1e3)
    e2e_value = tokens_per_step / (e2e_ms / 1e3)
    flops_per_token = trainer.metrics_processor.num_flops_per_token
    out = {
        "metric": "llama3_8b_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world), "dtype": "bf16",
        "data": "synthetic uniform tokens (seed 0), random-init weights",
        "config": {
            "model": "Llama-3.1-8B", "global_batch": local_bs * batch_degree, "seq_len": SEQ_LEN,
            "parallelism": parallelism,
            "per_op_sac_mm_policy": args.sac_mm_policy,
            "activation_checkpoint": f"{trainer.config.activation_checkpoint.mode}/{trainer.config.activation_checkpoint.selective_ac_option}"
                                     f" (matmul outputs kept: {_sac_mm_policy(trainer)})",
            "optimizer": "AdamW fused over flat shards, grad clip 1.0",
            "l2_between_iterations": "inputs and weights (16 GB bf16 + activations) exceed the 126 MB L2; no explicit flush",
            "per_gpu": {"tokens_per_sec": value / world, "mfu_pct_of_2.25PF": 100 * flops_per_token * value / world / 2.25e15,
                        "peak_reserved_gib": mem_gib},
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4, "last_loss": last_loss},
        "gpu_launches": int(launches),
        "kernel_error_flags": errs,
        "impl": "torchtitan_b200",
    }
    if args.kernel_table:
        write_kernel_table(args.kernel_table, lambda: step(host_iter), rank)
    if args.layers is not None:
        out["invalid_truncated_model_layers"] = args.layers
    if args.override:
        out["config"]["overrides"] = list(args.override)
    if args.config != "llama3_8b_synthetic":
        out["config"]["job_config"] = args.config
        out["dtype"] = "mxfp8 linears (bf16 elsewhere)" if "mxfp8" in args.config else out["dtype"]
    trainer.close()
    return out


def run_reference(args) -> dict:
    from baseline.run_reference import run as run_ref

    return run_ref(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--override", type=lambda v: v.split(), default=[], help="extra config flags for experiments as one "
                    "string, e.g. --override='--parallelism.fsdp_reshard_after_forward never' (recorded in the JSON line)")
    ap.add_argument("--layers", type=int, default=None, help="profiling aid: truncate the model (result is not a benchmark)")
    ap.add_argument("--ref-compile", action="store_true", help="reference arm only: time the --compile.enable build alone")
    ap.add_argument("--ref-build", default="both", choices=["both", "eager", "compile"],
                    help="reference arm only: which build(s) to time; 'both' reports the faster one")
    ap.add_argument("--config", default="llama3_8b_synthetic", help="job configuration of the llama3 module (e.g. "
                    "llama3_8b_synthetic_mxfp8); anything but the default is an experiment and is labelled in the output")
    ap.add_argument("--sac-mm-policy", default="every_second", choices=["every_second", "all", "auto"],
                    help="which matmul outputs per-op SAC keeps (every_second = the reference's policy)")
    ap.add_argument("--kernel-table", default=None, help="after the timed regions, run one more step under the PyTorch "
                    "profiler and write the device time per kernel name to this file")
    ap.add_argument("--ac", default=None, help="override activation_checkpoint.mode (selective|full|none)")
    args = ap.parse_args()
    assert args.warmup >= 3 or os.environ.get("TT_BENCH_ALLOW_SHORT_WARMUP"), "warm-up must be at least 3 steps"
    rank = int(os.environ.get("RANK", "0"))
    try:
        res = run_reference(args) if args.impl == "reference" else run_ours(args)
    except Exception as e:  # the reference arm must always answer with one line
        if args.impl == "reference":
            res = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        else:
            raise
    if rank == 0:
        print(json.dumps(res), flush=True)
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

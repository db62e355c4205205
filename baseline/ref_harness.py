"""Times the reference's own ``Trainer.train_step`` with the protocol of ``bench.py``."""

from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BASELINE_TOK_S_PER_GPU = 8307.5
SEQ_LEN = 8192


def run(args) -> dict:
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    if ROOT not in sys.path:
        sys.path.insert(1, ROOT)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    import torch
    import torch.distributed as dist

    import torchtitan
    assert os.path.realpath(torchtitan.__file__).startswith(os.path.realpath(os.path.join(HERE, "_ref"))), torchtitan.__file__
    from torchtitan.config.manager import ConfigManager
    from torchtitan.tools.logging import init_logger

    from bench import ClockSampler  # clock sampling helper only (no model code)

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    assert world == args.gpus
    if rank == 0:
        init_logger()
    total = args.warmup + 2 * args.steps + 4
    cli = ["--module", "baseline.ref_configs", "--config", "llama3_8b_synthetic", "--training.steps", str(total),
           "--dump_folder", "/tmp/tt_ref_bench", "--comm.train_timeout_seconds", "300"]
    if getattr(args, "ref_compile", False):
        cli += ["--compile.enable"]
    cfg = ConfigManager().parse_args(cli)
    trainer = cfg.build()
    dev = trainer.device
    bs = cfg.training.local_batch_size
    tokens_per_step = bs * SEQ_LEN * world
    host_iter = trainer.batch_generator(trainer.dataloader)

    def sync():
        if world > 1:
            dist.barrier(device_ids=[torch.cuda.current_device()])
        torch.cuda.synchronize()

    def max_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step(it):
        trainer.step += 1
        trainer.train_step(it)

    for _ in range(args.warmup):
        step(host_iter)
    sync()
    # the reference's train_step counts valid tokens on the host, so its batches must stay on the
    # CPU (pinned); its "device" region therefore already contains the 128 KiB host->device copy
    dit = host_iter
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(dit)
    e1.record()
    sync()
    dev_ms = max_ranks(e0.elapsed_time(e1)) / args.steps
    clocks = sampler.stop() if rank == 0 else {}
    # end to end: pinned host batches + the reference's own per-step loss read-out (log every step)
    trainer.metrics_processor.config.log_freq = 1
    sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        step(host_iter)
    f1.record()
    sync()
    e2e_ms = max_ranks(f0.elapsed_time(f1)) / args.steps
    if getattr(args, "kernel_table", None):
        from bench import write_kernel_table

        write_kernel_table(args.kernel_table, lambda: step(host_iter), rank)
    value = tokens_per_step / (dev_ms / 1e3)
    out = {
        "metric": "llama3_8b_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world), "dtype": "bf16",
        "data": "synthetic uniform tokens (seed 0), random-init weights",
        "config": {"model": "Llama-3.1-8B", "global_batch": bs * world, "seq_len": SEQ_LEN,
                   "parallelism": f"fsdp{world}" if world > 1 else "single-gpu (AMP)", "compile": bool(getattr(args, "ref_compile", False)),
                   "activation_checkpoint": "selective/op", "peak_reserved_gib": torch.cuda.max_memory_reserved() / 2**30,
                   "reference_version": getattr(torchtitan, "__version__", "?")},
        "clocks": clocks,
        "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 2 * bs * SEQ_LEN * 8, "d2h_bytes_per_step": 8},
        "gpu_launches": 0,
        "impl": "reference",
    }
    trainer.close()
    return out

"""Helpers to run a function on N CPU ranks (gloo) from a pytest test."""

from __future__ import annotations

import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    torch.set_num_threads(2)
    try:
        out = fn(rank, world, *args)
        torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
    except Exception:
        with open(os.path.join(result_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, tmp_path=None, timeout: int = 600):
    """Run ``fn(rank, world, *args)`` on ``world`` spawned CPU processes; return the list of results."""
    import tempfile

    result_dir = str(tmp_path) if tmp_path is not None else tempfile.mkdtemp()
    port = free_port()
    ctx = mp.spawn(_entry, args=(world, port, fn, args, result_dir), nprocs=world, join=False)
    import time

    t0 = time.time()
    while not ctx.join(timeout=5):
        if time.time() - t0 > timeout:
            for p in ctx.processes:
                p.terminate()
            raise TimeoutError("distributed test timed out")
    errs = [open(os.path.join(result_dir, f)).read() for f in os.listdir(result_dir) if f.endswith(".err")]
    if errs:
        raise RuntimeError("rank failed:\n" + "\n".join(errs))
    return [torch.load(os.path.join(result_dir, f"rank{r}.pt"), weights_only=False) for r in range(world)]

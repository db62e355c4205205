"""Load a model (optionally from a DCP checkpoint), generate from a prompt, report tokens/s and memory as JSON.

``python -m torchtitan_b200.scripts.generate.test_generate --module llama3 --config llama3_debugmodel
--checkpoint <dcp dir> --prompt "..." --max_new_tokens 32 [--temperature 0.8 --top_k 50 --seed 0 --out report.json]``.
With several ranks (``torchrun``) the model is tensor-parallel *without* sequence parallel (activations replicated), the
plan of scripts/generate/test_generate.py:40-70. Parity: scripts/generate/test_generate.py:72-330."""

from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from torchtitan_b200.config.manager import ConfigManager
from torchtitan_b200.tools.logging import init_logger, logger

from ._generation import generate


def apply_tp_minus_sp(model, tp_mesh) -> None:
    from torchtitan_b200.parallel.tp import apply_tp_to_decoder

    apply_tp_to_decoder(model, tp_mesh, loss_parallel=False, sequence_parallel=False)


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--module", default="llama3")
    ap.add_argument("--config", required=True)
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--max_new_tokens", type=int, default=32)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--top_k", type=int, default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    init_logger()
    config = ConfigManager().parse_args(["--module", a.module, "--config", a.config])
    if not a.prompt:
        logger.warning("The input prompt is empty, model will respond from a empty sequence.")
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device(f"cuda:{local_rank}") if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if a.deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
    tokenizer = config.tokenizer.build(tokenizer_path=config.hf_assets_path)
    model_config = config.model_spec.model
    model_config.update_from_config(trainer_config=config)
    with torch.device("meta" if world > 1 else device):
        model = model_config.build()
    if world > 1:
        from torchtitan_b200.parallel import ParallelDims

        dist.init_process_group("nccl" if device.type == "cuda" else "gloo")
        pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
        apply_tp_minus_sp(model, pd.get_mesh("tp"))
        model.to_empty(device=device)
    with torch.no_grad():
        model.init_weights(buffer_device=device)
    if device.type == "cuda":
        model.to(torch.bfloat16)
    model.eval()
    if a.checkpoint:
        import torch.distributed.checkpoint as dcp

        from torchtitan_b200.components.checkpoint import ModelWrapper
        from torchtitan_b200.parallel.tp import finalize_tp

        if world > 1:
            finalize_tp(model)                       # re-attach the sharding tags that to_empty() dropped
        wrapper = ModelWrapper(model)                # tensor-parallel shards appear with their full shape, as saved
        sd = wrapper.state_dict()
        t0 = time.monotonic()
        dcp.load(sd, checkpoint_id=a.checkpoint)
        wrapper.load_state_dict(sd)
        logger.info(f"Finished loading checkpoint in {time.monotonic() - t0:.2f} seconds.")
    ids = torch.tensor(tokenizer.encode(a.prompt, add_bos=True, add_eos=False), dtype=torch.long, device=device)
    ids = ids.view(1, -1).repeat(a.batch_size, 1)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.synchronize()
    t0 = time.monotonic()
    out = generate(model, ids, max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_k=a.top_k, seed=a.seed)
    if device.type == "cuda":
        torch.cuda.synchronize()
    dt = time.monotonic() - t0
    n_new = out.shape[1] - ids.shape[1]
    report = {
        "metadata": {"module": a.module, "config": a.config, "checkpoint": a.checkpoint, "world_size": world},
        "responses": [{"response_idx": i, "input_text": a.prompt, "output_text": tokenizer.decode(out[i, ids.shape[1]:].tolist())}
                      for i in range(out.shape[0])],
        "performance": {"generation_time_s": dt, "tokens_generated": n_new * out.shape[0], "tokens_per_s": n_new * out.shape[0] / dt},
        "memory": {"max_reserved_gib": torch.cuda.max_memory_reserved() / 2**30 if device.type == "cuda" else 0.0},
    }
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps(report, indent=2))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(report, f, indent=2)
    if dist.is_initialized():
        dist.destroy_process_group()
    return report


if __name__ == "__main__":
    main()

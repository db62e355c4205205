"""An analytic planner for B200 nodes and the bridge to the external ``autoparallel`` package.

The planner enumerates parallel layouts (data-parallel replicate x shard, tensor, pipeline, context and expert parallel,
FSDP reshard policy, activation checkpointing, pipeline schedule) for a model described by a handful of numbers, estimates
the peak memory per GPU and the step time of each from a roofline model of this framework on B200s, and returns the
fastest layout that fits. The constants are measurements of this framework, not data-sheet figures:

* dense bf16 work runs at 0.72 of the sustained cuBLAS rate inside a training step (Llama-3.1-8B, 1 GPU: 468.8 ms for
  4.74e14 FLOP);
* peer copies reach 770 GB/s per direction inside an NVSwitch node; between nodes a GPU is given 50 GB/s (one 400 Gb/s
  adapter), which is what makes the planner keep tensor, expert and shard groups inside a node;
* the FSDP gathers and reductions of one unit hide behind the compute of its neighbours as long as they take less time
  than that compute (weak scaling from 1 to 8 GPUs is flat); tensor-parallel collectives fused into the GEMMs hide about
  half of their wire time (FSDP 4 x TP 2: 655 ms per step against 489 ms for FSDP 8);
* selective (per-operation) checkpointing recomputes about 8 % of the forward FLOPs, full checkpointing all of them;
* mixture-of-experts steps reach 0.27 of the sustained rate on their active FLOPs (Qwen3-30B-A3B on 8 GPUs).

``python -m torchtitan_b200.experiments.autoparallel.planner --module llama3 --config llama3_70b --ngpu 64`` prints the
chosen layout with its command-line overrides and the runners-up.
"""

from __future__ import annotations

import argparse
import itertools
from dataclasses import dataclass, field

HBM_BYTES = 180e9
HBM_BW = 6.5e12               # measured copy bandwidth, bytes/s
NVLINK_BW = 770e9             # measured peer copy bandwidth per direction, bytes/s
INTERNODE_BW = 50e9           # one 400 Gb/s adapter per GPU
BF16_FLOPS = 1.4e15           # sustained dense bf16 (cuBLAS loop under the power cap)
STEP_EFFICIENCY = 0.72        # share of BF16_FLOPS a whole training step reaches (attention, norms, optimizer included)
MOE_STEP_EFFICIENCY = 0.27    # the same for mixture-of-experts models: routing, row gathers and many small expert GEMMs
                              # (Qwen3-30B-A3B, 8 GPUs, expert parallel 8: 10.3-12.0 k tokens/s/GPU)
GPUS_PER_NODE = 8
MEM_LIMIT = 0.92              # share of HBM a plan may use
AC_MEMORY = {"none": 1.0, "selective": 0.45, "full": 0.08}
AC_COMPUTE = {"none": 1.0, "selective": 1.0 + 0.08 / 3, "full": 1.0 + 1.0 / 3}   # forward is a third of a step's FLOPs


@dataclass
class ModelShape:
    """What the estimate needs to know about a model."""

    nparams: float                     # all parameters
    flops_per_token: float             # forward + backward FLOPs per token at ``seq_len``
    n_layers: int
    dim: int
    vocab_size: int = 128256
    expert_params: float = 0.0         # parameters inside routed experts (part of ``nparams``)
    num_experts: int = 0
    top_k: int = 0
    n_moe_layers: int = 0
    n_heads: int = 0                   # 0 = unknown; otherwise tensor parallel must divide both head counts
    n_kv_heads: int = 0

    @property
    def dense_params(self) -> float:
        return self.nparams - self.expert_params


@dataclass
class Plan:
    dp_shard: int
    tp: int
    reshard_after_forward: str
    ac_mode: str
    est_step_s: float
    est_mem_bytes: float
    dp_replicate: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    pp_schedule: str = "1F1B"
    n_microbatches: int = 1
    breakdown: dict = field(default_factory=dict)

    @property
    def world_size(self) -> int:
        return self.dp_replicate * self.dp_shard * self.cp * self.tp * self.pp

    def tokens_per_second(self, seq_len: int, local_batch: int) -> float:
        return seq_len * local_batch * self.dp_replicate * self.dp_shard / self.est_step_s

    def to_overrides(self) -> list[str]:
        out = [f"--parallelism.data_parallel_replicate_degree={self.dp_replicate}",
               f"--parallelism.data_parallel_shard_degree={self.dp_shard}", f"--parallelism.tensor_parallel_degree={self.tp}",
               f"--parallelism.fsdp_reshard_after_forward={self.reshard_after_forward}", f"--activation_checkpoint.mode={self.ac_mode}"]
        if self.cp > 1:
            out.append(f"--parallelism.context_parallel_degree={self.cp}")
        if self.ep > 1:
            out.append(f"--parallelism.expert_parallel_degree={self.ep}")
        if self.pp > 1:
            out += [f"--parallelism.pipeline_parallel_degree={self.pp}", f"--parallelism.pipeline_parallel_schedule={self.pp_schedule}"]
        if self.tp > 1:
            out.append("--parallelism.enable_async_tensor_parallel")
        return out

    def describe(self) -> str:
        dims = [f"dp_replicate={self.dp_replicate}", f"dp_shard={self.dp_shard}", f"cp={self.cp}", f"tp={self.tp}",
                f"pp={self.pp}" + (f" ({self.pp_schedule}, {self.n_microbatches} micro-batches)" if self.pp > 1 else ""),
                f"ep={self.ep}", f"ac={self.ac_mode}", f"reshard={self.reshard_after_forward}"]
        parts = ", ".join(f"{k} {v * 1e3:.0f} ms" for k, v in self.breakdown.items() if v > 5e-4)
        return (f"{' '.join(dims)}: {self.est_step_s * 1e3:.0f} ms/step, {self.est_mem_bytes / 1e9:.0f} GB/GPU" +
                (f" [{parts}]" if parts else ""))


def _bw(group_span: int, gpus_per_node: int) -> float:
    """Bandwidth per GPU of a collective whose group covers ``group_span`` consecutive ranks."""
    return NVLINK_BW if group_span <= gpus_per_node else INTERNODE_BW


def estimate(m: ModelShape, seq_len: int, local_batch: int, *, dp_replicate: int, dp_shard: int, cp: int, tp: int, pp: int, ep: int,
             reshard: str, ac: str, schedule: str = "1F1B", gpus_per_node: int = GPUS_PER_NODE) -> tuple[float, float, dict, int]:
    """(step seconds, peak bytes per GPU, time breakdown, micro-batches) of one layout. ``local_batch`` is the number of
    sequences per data-parallel rank and step."""
    layers = m.n_layers / pp
    tokens = seq_len * local_batch                       # per data-parallel rank
    tokens_gpu = tokens / (cp * tp)                      # activations held per GPU (sequence parallel shards them over tp)
    fsdp = dp_shard * cp                                 # ranks the dense parameters are sharded over
    efsdp = max(1, fsdp * tp // max(ep, 1))              # and the experts, beside ep
    # ---- memory --------------------------------------------------------------------------------------------------------
    dense_local = m.dense_params / (tp * pp)
    expert_local = m.expert_params / (max(ep, 1) * pp)
    mem = 16.0 * (dense_local / fsdp + expert_local / efsdp)              # fp32 master, two moments, fp32 gradient shard
    per_layer = 2.0 * (dense_local + expert_local) / max(layers, 1)
    mem += 2.0 * (dense_local + expert_local) if (reshard == "never" and fsdp > 1) else 3 * per_layer   # bf16 gathered copies
    n_mb = 1
    in_flight = 1.0
    if pp > 1:
        n_mb = max(1, min(local_batch, 2 * pp))
        in_flight = min(n_mb, pp) / n_mb                 # share of the local batch whose activations are alive at once
    act_layer = 34.0 * m.dim                             # bytes per token and layer kept for backward without checkpointing
    mem += act_layer * tokens_gpu * layers * AC_MEMORY[ac] * in_flight
    mem += 6.0 * (tokens / cp) * m.vocab_size / tp / n_mb    # logits of one micro-batch: bf16 + an fp32 chunk (loss parallel)
    mem += 2e9                                           # context, workspaces, collective buffers
    # ---- time ----------------------------------------------------------------------------------------------------------
    efficiency = MOE_STEP_EFFICIENCY if m.expert_params else STEP_EFFICIENCY
    compute = m.flops_per_token * tokens / (cp * tp * pp) * AC_COMPUTE[ac] / (BF16_FLOPS * efficiency)
    shard_span = fsdp * tp                               # tp is innermost, then the shard dimension
    gather_bytes = 2.0 * dense_local * (fsdp - 1) / fsdp + 2.0 * expert_local * (efsdp - 1) / efsdp
    n_gathers = 2 if reshard == "never" else 3           # forward gather (+ backward re-gather) + gradient reduce-scatter
    fsdp_wire = n_gathers * gather_bytes / _bw(shard_span, gpus_per_node) if fsdp > 1 else 0.0
    fsdp_exposed = max(0.0, fsdp_wire - 0.9 * compute)
    replicate_wire = 2 * 4.0 * (dense_local / fsdp + expert_local / efsdp) / _bw(dp_replicate * shard_span, gpus_per_node) \
        if dp_replicate > 1 else 0.0
    replicate_exposed = max(0.0, replicate_wire - 0.5 * compute)
    tp_wire = 0.0
    if tp > 1:
        # per layer: 2 all-gathers + 2 reduce-scatters of the [tokens, dim] activations forward, the same backward
        tp_wire = 8 * layers * 2.0 * (tokens / cp) * m.dim * (tp - 1) / tp / _bw(tp, gpus_per_node)
    tp_exposed = 0.5 * tp_wire
    cp_exposed = 0.0
    if cp > 1:
        kv = 2 * 2.0 * (tokens / cp) * m.dim / 4         # K and V of a grouped-query model, per ring step
        cp_wire = 3 * layers * kv * (cp - 1) / _bw(cp * tp, gpus_per_node)
        cp_exposed = max(0.0, cp_wire - 0.3 * compute) + 0.03 * compute        # head-tail balancing overhead
    ep_exposed = 0.0
    if ep > 1 and m.n_moe_layers:
        rows = tokens_gpu * m.top_k * m.dim * 2.0        # bytes dispatched per MoE layer and direction
        ep_wire = 4 * (m.n_moe_layers / pp) * rows * (ep - 1) / ep / _bw(ep * tp, gpus_per_node)
        ep_exposed = ep_wire                             # the exchange sits between the router and the expert GEMMs
    bubble = 0.0
    if pp > 1:
        ideal = (pp - 1) / (n_mb + pp - 1)
        # two stages per rank halve the 1F1B bubble; split backward steps fill about two thirds of it, down to the few
        # percent the list scheduler reaches at 2 x pp micro-batches
        share = {"1F1B": ideal, "Interleaved1F1B": ideal / 2, "ZBVZeroBubble": max(0.04, ideal / 3),
                 "InterleavedZeroBubble": max(0.05, ideal / 3), "DualPipeV": max(0.04, ideal / 3)}.get(schedule, ideal)
        bubble = compute * share / (1 - share)
        bubble += n_mb * 4 * 2.0 * tokens_gpu / n_mb * m.dim / _bw(world_span(dp_replicate, fsdp, tp, pp), gpus_per_node)
    optimizer = 16.0 * (dense_local / fsdp + expert_local / efsdp) * 1.25 / HBM_BW
    parts = {"compute": compute, "fsdp": fsdp_exposed, "replicate": replicate_exposed, "tp": tp_exposed, "cp": cp_exposed,
             "ep": ep_exposed, "pipeline": bubble, "optimizer": optimizer}
    return sum(parts.values()), mem, parts, n_mb


def world_span(dp_replicate: int, fsdp: int, tp: int, pp: int) -> int:
    """Consecutive ranks one pipeline hop skips: pipeline stages are the outermost dimension."""
    return dp_replicate * fsdp * tp * (2 if pp > 1 else 1)


def _divisors(n: int, limit: int) -> list[int]:
    return [d for d in (1, 2, 4, 8, 16, 32, 64) if d <= limit and n % d == 0]


def search(m: ModelShape, seq_len: int, local_batch: int, world_size: int, gpus_per_node: int = GPUS_PER_NODE,
           keep: int = 5) -> list[Plan]:
    """The ``keep`` fastest layouts (per globally processed token) that fit in memory, best first."""
    plans: list[Plan] = []
    moe = m.num_experts > 0
    for tp, pp, cp in itertools.product(_divisors(world_size, gpus_per_node), _divisors(world_size, world_size),
                                        _divisors(world_size, gpus_per_node)):
        if world_size % (tp * pp * cp) or m.n_layers % pp or (pp > 1 and m.n_layers // pp < 1):
            continue
        if (m.n_heads and m.n_heads % tp) or (m.n_kv_heads and m.n_kv_heads % tp):
            continue
        if seq_len % (2 * cp * tp) or (cp > 1 and seq_len < 16384):
            continue                                     # context parallel pays off on long sequences only
        dp = world_size // (tp * pp * cp)
        for dp_replicate in _divisors(dp, dp):
            dp_shard = dp // dp_replicate
            if dp_replicate > 1 and dp_shard * cp * tp < min(gpus_per_node, world_size // pp):
                continue                                 # replicate only across nodes, shard inside
            eps = [e for e in _divisors(m.num_experts, dp_shard * cp * tp) if (dp_shard * cp * tp) % e == 0] if moe else [1]
            for ep in eps:
                schedules = ["1F1B"] if pp == 1 else ["1F1B", "Interleaved1F1B", "ZBVZeroBubble"] + (["DualPipeV"] if ep > 1 else [])
                for reshard, ac, schedule in itertools.product(("never", "always"), ("none", "selective", "full"), schedules):
                    if schedule != "1F1B" and m.n_layers % (2 * pp):
                        continue                         # two stages per rank
                    t, mem, parts, n_mb = estimate(m, seq_len, local_batch, dp_replicate=dp_replicate, dp_shard=dp_shard, cp=cp,
                                                   tp=tp, pp=pp, ep=ep, reshard=reshard, ac=ac, schedule=schedule,
                                                   gpus_per_node=gpus_per_node)
                    if mem > MEM_LIMIT * HBM_BYTES:
                        continue
                    plans.append(Plan(dp_shard, tp, reshard, ac, t, mem, dp_replicate=dp_replicate, pp=pp, cp=cp, ep=ep,
                                      pp_schedule=schedule, n_microbatches=n_mb, breakdown=parts))
    # time per globally processed token; ties go to the simpler layout (fewer model-parallel dimensions, less recompute)
    plans.sort(key=lambda p: (round(p.est_step_s / (p.dp_replicate * p.dp_shard), 6), p.tp * p.pp * p.cp, p.est_mem_bytes))
    out, seen = [], set()
    for p in plans:
        key = (p.dp_replicate, p.dp_shard, p.tp, p.pp, p.cp, p.ep)
        if key in seen:
            continue
        seen.add(key)
        out.append(p)
        if len(out) == keep:
            break
    return out


def auto_plan(nparams: float, flops_per_token: float, n_layers: int, dim: int, seq_len: int, local_batch: int, world_size: int,
              *, vocab_size: int = 128256, expert_params: float = 0.0, num_experts: int = 0, top_k: int = 0, n_moe_layers: int = 0,
              n_heads: int = 0, n_kv_heads: int = 0, gpus_per_node: int = GPUS_PER_NODE) -> Plan:
    """Cheapest estimated step per processed token among the layouts that fit in memory."""
    shape = ModelShape(nparams, flops_per_token, n_layers, dim, vocab_size, expert_params, num_experts, top_k, n_moe_layers,
                       n_heads, n_kv_heads)
    found = search(shape, seq_len, local_batch, world_size, gpus_per_node, keep=1)
    if not found:
        raise RuntimeError("no plan fits in memory on these GPUs; add nodes")
    return found[0]


def shape_of(model_config, model, seq_len: int) -> ModelShape:
    """``ModelShape`` of a decoder configuration and its (meta-device) model."""
    nparams, flops = model_config.get_nparams_and_flops(model, seq_len)
    expert = sum(p.numel() for n, p in model.named_parameters() if ".experts." in n)
    moe_layers = len({n.split(".experts.")[0] for n, _ in model.named_parameters() if ".experts." in n})
    layer = getattr(model_config, "layer", None)
    moe, attn = getattr(layer, "moe", None), getattr(layer, "attention", None)
    heads = getattr(attn, "n_heads", 0) or 0
    return ModelShape(float(sum(p.numel() for p in model.parameters())), float(flops), model_config.n_layers, model_config.dim,
                      getattr(model_config, "vocab_size", 128256), float(expert), getattr(moe, "num_experts", 0) if expert else 0,
                      getattr(moe, "top_k", 0) if expert else 0, moe_layers, heads, getattr(attn, "n_kv_heads", None) or heads)


def parallelize_with_autoparallel(model, mesh, input_fn, **kwargs):
    """Delegate to the external package when it is installed (same call the reference experiment makes)."""
    try:
        from autoparallel.api import AutoParallel  # type: ignore
    except ImportError as e:
        raise ImportError("the 'autoparallel' package is not installed; use experiments.autoparallel.auto_plan "
                          "for the built-in planner") from e
    with AutoParallel(model, input_fn, mesh, **kwargs) as autop:
        autop.add_parameter_memory_constraint(low=None, high=None)
        placement = autop.optimize_placement()
        return autop.apply_placement(placement)


def main(argv: list[str] | None = None) -> int:
    import torch

    from torchtitan_b200.config.manager import ConfigManager

    ap = argparse.ArgumentParser(description="Plan a parallel layout for a job configuration.")
    ap.add_argument("--module", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--ngpu", type=int, default=8)
    ap.add_argument("--gpus_per_node", type=int, default=GPUS_PER_NODE)
    ap.add_argument("--seq_len", type=int, default=None)
    ap.add_argument("--local_batch_size", type=int, default=None)
    a = ap.parse_args(argv)
    cfg = ConfigManager().parse_args(["--module", a.module, "--config", a.config])
    seq = a.seq_len or cfg.training.seq_len
    batch = a.local_batch_size or cfg.training.local_batch_size
    mc = cfg.model_spec.model
    with torch.device("meta"):
        model = mc.build()
    shape = shape_of(mc, model, seq)
    plans = search(shape, seq, batch, a.ngpu, a.gpus_per_node)
    if not plans:
        print("no layout fits in memory; add nodes")
        return 1
    print(f"{a.module}/{a.config}: {shape.nparams / 1e9:.1f} B parameters ({shape.expert_params / 1e9:.1f} B in experts), "
          f"{seq} tokens x {batch} per data-parallel rank, {a.ngpu} GPUs")
    for i, p in enumerate(plans):
        print(("* " if i == 0 else "  ") + p.describe() + f"  -> {p.tokens_per_second(seq, batch) / a.ngpu:,.0f} tok/s/GPU")
    print(" ".join(plans[0].to_overrides()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

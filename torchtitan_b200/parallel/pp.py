"""Pipeline parallelism: FQN-based stage split, schedules and the P2P runtime.

What it reproduces from torchtitan/distributed/pipeline_parallel.py:48-513: the model is split by
fully-qualified module names (``module_fqns_per_model_part`` or an automatic layout in which the
embedding and the output layer count as ``first/last_stage_less_layers`` layers), every stage is a
deep copy of the meta model with the other modules removed (``layers`` keeps its string keys,
missing top-level modules become ``None`` and are skipped by ``Decoder.forward``), stages are placed
on ranks in loop order (``stage = rank + i * pp``) or V order for ``ZBVZeroBubble`` / ``DualPipeV``,
each stage is parallelised with the model's own ``parallelize_fn``, and
``n_microbatches = local_batch_size / pipeline_parallel_microbatch_size``.

The runtime is this framework's own (the reference uses ``torch.distributed.pipelining``): a
schedule is a per-rank list of actions ``(stage, F|B, microbatch)``; activations and their gradients
travel by asynchronous NCCL/gloo point-to-point messages; every stage output keeps its autograd graph
until its backward action. Schedules: ``GPipe``, ``1F1B``, ``Interleaved1F1B`` / ``LoopedBFS`` (two or
more stages per rank), ``InterleavedZeroBubble``, ``ZBVZeroBubble`` and ``DualPipeV`` (the last two with V
placement), and CSV files with one line of actions per rank (``0F0,0F1,0I0,0W0,...``).

Zero-bubble schedules split a backward step into ``I`` (gradient of the stage input, sent on at once) and ``W`` (the
weight gradients of the stage's linear layers, parked by ``ops/wgrad_store.py`` and run where the rank would wait for
a message). The split needs weights that own their ``.grad`` (pipeline-only or pipeline x tensor parallel); stages
under FSDP or replicate units, whose reduce-scatter consumes the weight gradients inside the backward pass, run the
same placement with whole ``B`` steps and say so at start-up.
"""

from __future__ import annotations

import copy
import csv
import math
import re
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from torchtitan_b200.ops.wgrad_store import WeightGradStore
from torchtitan_b200.tools.logging import logger

__all__ = ["pipeline_llm", "generate_llm_fqn_per_model_part", "pipeline_module_split", "PipelineSchedule",
           "build_actions", "SCHEDULES"]

SINGLE_STAGE = {"GPipe", "1F1B"}
MULTI_STAGE = {"Interleaved1F1B", "LoopedBFS", "InterleavedZeroBubble", "ZBVZeroBubble", "DualPipeV"}
V_STYLE = {"ZBVZeroBubble", "DualPipeV"}
ZERO_BUBBLE = {"InterleavedZeroBubble", "ZBVZeroBubble", "DualPipeV"}
SCHEDULES = SINGLE_STAGE | MULTI_STAGE


# ------------------------------------------------------------------------------------ stage layout
def generate_llm_fqn_per_model_part(num_stages: int, num_layers: int, input_weight: int = 1, output_weight: int = 1):
    """Split ``tok_embeddings, layers.0..L-1, norm, output`` into ``num_stages`` FQN lists; the
    embedding weighs ``input_weight`` layers and norm+output ``output_weight`` layers."""
    if num_stages < 1:
        raise ValueError("Number of stages must be at least 1")
    if num_stages == 1:
        return [["tok_embeddings"] + [f"layers.{i}" for i in range(num_layers)] + ["norm", "output"]]
    effective = num_layers + input_weight + output_weight
    if num_stages > effective:
        raise ValueError(f"Number of stages ({num_stages}) cannot be greater than effective layers ({effective})")
    base, extra = divmod(effective, num_stages)
    if base <= input_weight and num_stages > 1 and base < input_weight:
        raise ValueError(f"Not enough layers for the first stage: {base} per stage vs input weight {input_weight}")
    if output_weight > base:
        raise ValueError(f"output_weight ({output_weight}) exceeds minimum layers per stage ({base}).")
    out, cur = [], 0
    for s in range(num_stages):
        budget = base + (1 if s < extra else 0)
        names = []
        if s == 0:
            names.append("tok_embeddings")
            budget -= input_weight
        if s == num_stages - 1:
            budget -= output_weight
        budget = max(budget, 0)
        if s == num_stages - 1:
            budget = num_layers - cur
        for _ in range(budget):
            if cur < num_layers:
                names.append(f"layers.{cur}")
                cur += 1
        if s == num_stages - 1:
            names += ["norm", "output"]
        out.append(names)
    return out


def _build_stage(whole: nn.Module, fqns: list[str]) -> nn.Module:
    if hasattr(whole, "build_pipeline_stage"):       # models whose parts are not direct children build their own stage
        return whole.build_pipeline_stage(fqns)
    model = copy.deepcopy(whole)
    keep = set(fqns)
    for name, child in list(model.named_children()):
        if isinstance(child, (nn.ModuleDict, nn.ModuleList)):
            wanted = {f.split(".", 1)[1] for f in keep if f.startswith(name + ".")}
            if isinstance(child, nn.ModuleDict):
                for k in list(child.keys()):
                    if k not in wanted:
                        del child[k]
            else:
                setattr(model, name, nn.ModuleList([m for i, m in enumerate(child) if str(i) in wanted]))
        elif name not in keep:
            setattr(model, name, None)
    return model


def stage_indices_for_rank(pp_rank: int, pp: int, num_stages: int, style: str) -> tuple[int, ...]:
    per = num_stages // pp
    if style == "loop":
        return tuple(pp_rank + s * pp for s in range(per))
    assert per == 2, f"v schedules assume 2 stages per rank, got {per}"
    return (pp_rank, num_stages - 1 - pp_rank)


def stage_to_rank(stage: int, pp: int, num_stages: int, style: str) -> int:
    if style == "loop":
        return stage % pp
    return stage if stage < pp else num_stages - 1 - stage


def pipeline_module_split(whole: nn.Module, pp_rank: int, pp: int, schedule: str, module_names_per_stage):
    style = "v" if schedule in V_STYLE else "loop"
    num_stages = len(module_names_per_stage)
    idx = stage_indices_for_rank(pp_rank, pp, num_stages, style)
    parts = [_build_stage(whole, module_names_per_stage[i]) for i in idx]
    for i in idx:
        logger.info(f"PP rank {pp_rank} is building stage_idx {i} with modules {module_names_per_stage[i]}")
    return idx, parts, style


# ------------------------------------------------------------------------------------ schedules
@dataclass(frozen=True)
class Action:
    stage: int
    kind: str  # "F" forward, "B" whole backward, "I" input-gradient half, "W" weight-gradient half, "O" overlapped pair
    mb: int
    other: tuple | None = None  # kind "O": (stage, mb) name the forward, ``other`` = (kind "B" | "I", stage, mb) the backward

    def parts(self) -> list["Action"]:
        """The plain actions this one stands for (an overlapped pair is its forward, then its backward)."""
        if self.kind != "O":
            return [self]
        return [Action(self.stage, "F", self.mb), Action(self.other[1], self.other[0], self.other[2])]


def _parse_action(tok: str) -> Action:
    tok = tok.strip()
    pair = re.fullmatch(r"(\d+)F(\d+)\+(\d+)([BI])(\d+)", tok)       # a forward and a backward in one slot: 0F4+7B1
    if pair:
        return Action(int(pair.group(1)), "O", int(pair.group(2)), (pair.group(4), int(pair.group(3)), int(pair.group(5))))
    m = re.fullmatch(r"(\d+)([FBIW]|BW)(\d+)", tok)
    if not m:
        raise ValueError(f"cannot parse pipeline action '{tok}'")
    kind = m.group(2)
    if kind == "BW":
        kind = "B"
    return Action(int(m.group(1)), kind, int(m.group(3)))


def load_csv_actions(path: str) -> list[list[Action]]:
    rows = []
    with open(path, newline="") as f:
        for row in csv.reader(f):
            rows.append([_parse_action(t) for t in row if t.strip()])
    return rows


def fuse_split_backward(ranks: list[list[Action]]) -> list[list[Action]]:
    """The same schedule with whole backward steps: ``I`` becomes ``B`` and ``W`` is dropped."""
    def whole(a):
        if a.kind == "I":
            return Action(a.stage, "B", a.mb)
        if a.kind == "O" and a.other[0] == "I":
            return Action(a.stage, "O", a.mb, ("B", a.other[1], a.other[2]))
        return a

    return [[whole(a) for a in acts if a.kind != "W"] for acts in ranks]


def pair_forward_backward(ranks: list[list[Action]], pp: int, num_stages: int, n_mb: int, style: str,
                          credit: float = 0.15) -> list[list[Action]]:
    """DualPipeV's overlapped slots: a forward next to a backward (or input-gradient) step of a different micro-batch on
    the same rank become one action whose two halves run together (``parallel/overlap.py``). Both halves take their
    inputs before either sends its output (the two sends leave in a fixed order, whichever half finishes first), so a
    pair is kept only if the dependency simulation still completes with it: candidates are tried one by one."""
    out = [list(acts) for acts in ranks]
    limit = estimate_makespan(out, num_stages)[0]          # a pairing must pay for the waiting it adds
    for r in range(len(out)):
        i = 0
        while i + 1 < len(out[r]):
            a, b = out[r][i], out[r][i + 1]
            if a.mb != b.mb and {a.kind, b.kind} in ({"F", "B"}, {"F", "I"}):
                f, bk = (a, b) if a.kind == "F" else (b, a)
                trial = out[r][:i] + [Action(f.stage, "O", f.mb, (bk.kind, bk.stage, bk.mb))] + out[r][i + 2:]
                keep = out[r]
                out[r] = trial
                try:
                    validate_actions(out, pp, num_stages, n_mb, style)
                    t = estimate_makespan(out, num_stages, pair_credit=credit)[0]
                    if t > limit:
                        out[r] = keep
                    else:
                        limit = t
                except RuntimeError:
                    out[r] = keep
            i += 1
    return out


def split_backward(ranks: list[list[Action]], pp: int, style: str) -> list[list[Action]]:
    """Turn every ``B`` into ``I`` plus a later ``W``. A rank keeps up to ``lag`` weight-gradient steps in hand and
    runs the oldest after each ``I`` beyond that, so in the cool-down (where a rank waits for the next gradient after
    every ``I``) one ``W`` fills each wait, and the rest run at the end instead of the idle tail. ``lag`` is the number
    of ranks behind this one in the backward direction (``pp - 1 - rank``) for loop placement and ``pp - 1`` for V
    placement, where every rank holds both an early and a late stage."""
    out = []
    for r, acts in enumerate(ranks):
        lag = (pp - 1 - r) if style == "loop" else (pp - 1)
        res, backlog = [], []
        for a in acts:
            if a.kind != "B":
                res.append(a)
                continue
            res.append(Action(a.stage, "I", a.mb))
            backlog.append(Action(a.stage, "W", a.mb))
            if len(backlog) > lag:
                res.append(backlog.pop(0))
        out.append(res + backlog)
    return out


def list_schedule(pp: int, num_stages: int, n_mb: int, style: str, slack: int = 1, split: bool = True) -> list[list[Action]]:
    """Pipeline order by list scheduling on a unit-time grid: a forward and each backward half take one tick, a whole
    backward two. With ``split`` a backward is an ``I`` step plus a parked ``W`` step (zero-bubble order), otherwise
    one ``B`` step. A free rank prefers, in this order: a backward (input-gradient) step whose gradient has arrived (it
    unblocks the rank before it; deepest local stage first), a weight-gradient step once more than ``pp`` of them are
    parked (bounds the activations they hold), a forward step (deepest local stage first, so a micro-batch reaches the
    loss as early as possible) while the stage has fewer than ``slack * ceil(2 (S - s) / (3 L)) + 1`` micro-batches
    in flight (``S`` stages, ``L`` per rank: the round trip from stage ``s`` to the loss and back over the time a rank
    spends per micro-batch), and otherwise a parked weight-gradient step: that is what fills the waits of the warm-up
    and cool-down phases. The oldest micro-batch in flight is never held by a cap (a stage works in order, so the
    stage it waits at holds nothing newer), hence the loop always makes progress."""
    my_stages = [stage_indices_for_rank(r, pp, num_stages, style) for r in range(pp)]
    n_local = len(my_stages[0])
    done_at: dict = {}                                    # (stage, "F" | "B", mb) -> first tick at which the result exists
    ranks: list[list[Action]] = [[] for _ in range(pp)]
    next_f = [{s: 0 for s in my_stages[r]} for r in range(pp)]
    next_b = [{s: 0 for s in my_stages[r]} for r in range(pp)]
    parked: list[list[Action]] = [[] for _ in range(pp)]
    busy_until = [0] * pp
    inflight = {s: 0 for st in my_stages for s in st}
    cap = {s: slack * math.ceil(2 * (num_stages - s) / (3 * n_local)) + 1 for s in inflight}
    total = sum((3 if split else 2) * n_mb * len(st) for st in my_stages)
    emitted, t = 0, 0
    never = 1 << 60
    while emitted < total:
        for r in range(pp):
            if busy_until[r] > t:
                continue
            pick = None
            for st in sorted(my_stages[r], reverse=True):
                m = next_b[r][st]
                if m < n_mb and done_at.get((st, "F", m), never) <= t and \
                        (st == num_stages - 1 or done_at.get((st + 1, "B", m), never) <= t):
                    pick = Action(st, "I" if split else "B", m)
                    break
            if pick is None and len(parked[r]) > pp:
                pick = parked[r][0]
            if pick is None:
                for st in sorted(my_stages[r], reverse=True):
                    m = next_f[r][st]
                    if m < n_mb and inflight[st] < cap[st] and (st == 0 or done_at.get((st - 1, "F", m), never) <= t):
                        pick = Action(st, "F", m)
                        break
            if pick is None and parked[r]:
                pick = parked[r][0]
            if pick is None:
                continue
            ranks[r].append(pick)
            emitted += 1
            busy_until[r] = t + (2 if pick.kind == "B" else 1)
            if pick.kind == "F":
                done_at[(pick.stage, "F", pick.mb)] = busy_until[r]
                next_f[r][pick.stage] += 1
                inflight[pick.stage] += 1
            elif pick.kind == "W":
                parked[r].pop(0)
            else:
                done_at[(pick.stage, "B", pick.mb)] = busy_until[r]
                next_b[r][pick.stage] += 1
                inflight[pick.stage] -= 1
                if split:
                    parked[r].append(Action(pick.stage, "W", pick.mb))
        t += 1
        if t > 16 * total + 64:
            raise RuntimeError("pipeline list scheduling made no progress")
    return ranks


def _shortest(candidates: list, num_stages: int):
    return min(candidates, key=lambda acts: estimate_makespan(acts, num_stages)[0])     # ties: the earlier candidate


def build_actions(schedule: str, pp: int, num_stages: int, n_mb: int, style: str = "loop",
                  split: bool = False, overlap: bool = False) -> list[list[Action]]:
    """Per-rank ordered action lists. ``split`` gives a zero-bubble schedule separate I / W steps. The zero-bubble
    schedules take the shortest (by :func:`estimate_makespan`) of the interleaved-1F1B-derived order and two list-scheduled
    orders (in-flight slack 1 to 3; more slack holds more activations, and ties go to less). ``overlap`` (DualPipeV
    only) merges forward / backward neighbours of different micro-batches into slots that run both at once."""
    if schedule in ZERO_BUBBLE:
        base = build_actions("Interleaved1F1B", pp, num_stages, n_mb, style)
        if split:
            base = split_backward(base, pp, style)
        best = _shortest([base] + [list_schedule(pp, num_stages, n_mb, style, k, split) for k in (1, 2, 3)], num_stages)
        return pair_forward_backward(best, pp, num_stages, n_mb, style) if (overlap and schedule == "DualPipeV") else best
    ranks: list[list[Action]] = [[] for _ in range(pp)]
    my_stages = [stage_indices_for_rank(r, pp, num_stages, style) for r in range(pp)]
    if schedule == "GPipe":
        for r in range(pp):
            s = my_stages[r][0]
            ranks[r] = [Action(s, "F", m) for m in range(n_mb)] + [Action(s, "B", m) for m in range(n_mb)]
        return ranks
    if schedule == "1F1B":
        for r in range(pp):
            s = my_stages[r][0]
            warm = min(pp - r, n_mb)
            acts = [Action(s, "F", m) for m in range(warm)]
            f, b = warm, 0
            while b < n_mb:
                acts.append(Action(s, "B", b)); b += 1
                if f < n_mb:
                    acts.append(Action(s, "F", f)); f += 1
            ranks[r] = acts
        return ranks
    # multi-stage schedules: breadth-first rounds of pp micro-batches per local stage (interleaved 1F1B order
    # for the forward sweep, mirrored for backward); correct for loop and V placement.
    for r in range(pp):
        stages = my_stages[r]
        fwd = []
        for m0 in range(0, n_mb, pp):
            for s in stages:
                for m in range(m0, min(m0 + pp, n_mb)):
                    fwd.append(Action(s, "F", m))
        bwd = []
        for m0 in range(0, n_mb, pp):
            for s in reversed(stages):
                for m in range(m0, min(m0 + pp, n_mb)):
                    bwd.append(Action(s, "B", m))
        if schedule == "LoopedBFS":
            ranks[r] = fwd + bwd
            continue
        # 1F1B steady state: after a warm-up of forwards alternate one backward / one forward
        n_local = len(stages)
        warm = min(len(fwd), (n_local - 1) * pp + 2 * (pp - 1 - r) + 1) if style == "loop" else min(len(fwd), n_local * pp)
        acts = fwd[:warm]
        fi, bi = warm, 0
        while bi < len(bwd):
            acts.append(bwd[bi]); bi += 1
            if fi < len(fwd):
                acts.append(fwd[fi]); fi += 1
        ranks[r] = acts
    return ranks


def validate_actions(ranks: list[list[Action]], pp: int, num_stages: int, n_mb: int, style: str) -> None:
    """Simulate the schedule with blocking receives and asynchronous sends; raise on deadlock."""
    done = set()
    pos = [0] * len(ranks)
    progressed = True
    while progressed:
        progressed = False
        for r, acts in enumerate(ranks):
            while pos[r] < len(acts):
                a = acts[pos[r]]
                if a.kind == "O":
                    # both halves take their inputs before either sends its output
                    bk, bs, bm = a.other
                    ready = (a.stage == 0 or (a.stage - 1, "F", a.mb) in done) and (bs, "F", bm) in done and \
                        (bs == num_stages - 1 or (bs + 1, "B", bm) in done)
                    if not ready:
                        break
                    done.update({(a.stage, "F", a.mb), (bs, bk, bm), (bs, "B", bm)})
                    pos[r] += 1
                    progressed = True
                    continue
                if a.kind == "F":
                    ready = a.stage == 0 or (a.stage - 1, "F", a.mb) in done
                elif a.kind == "W":
                    if (a.stage, "I", a.mb) not in done:
                        raise RuntimeError(f"pipeline schedule: {a.stage}W{a.mb} on rank {r} comes before its {a.stage}I{a.mb}")
                    ready = True
                else:                                    # "B" and "I" both deliver the input gradient, recorded as "B"
                    ready = (a.stage, "F", a.mb) in done and (a.stage == num_stages - 1 or (a.stage + 1, "B", a.mb) in done)
                if not ready:
                    break
                done.add((a.stage, a.kind, a.mb))
                if a.kind == "I":
                    done.add((a.stage, "B", a.mb))
                pos[r] += 1
                progressed = True
    if any(pos[r] < len(ranks[r]) for r in range(len(ranks))):
        raise RuntimeError(f"pipeline schedule deadlocks: progress {pos} of {[len(a) for a in ranks]}")
    flat = [b for acts in ranks for a in acts for b in a.parts()]
    owed = {(a.stage, a.mb) for a in flat if a.kind == "I"} - {(a.stage, a.mb) for a in flat if a.kind == "W"}
    if owed:
        raise RuntimeError(f"pipeline schedule: input-gradient steps without a weight-gradient step: {sorted(owed)[:4]}")


def estimate_makespan(ranks: list[list[Action]], num_stages: int, cost: dict | None = None,
                      pair_credit: float = 0.0) -> tuple[float, float]:
    """Length of one step and the idle fraction of the busiest-possible timeline, from a dependency simulation with
    per-action costs (default: a forward 1, a whole backward 2, each backward half 1; messages are free). An overlapped
    pair starts when the inputs of both halves are there, takes the sum of their costs less ``pair_credit`` of it (the
    share of a slot that the overlapped exchanges are expected to hide) and delivers both outputs at its end."""
    cost = cost or {"F": 1.0, "B": 2.0, "I": 1.0, "W": 1.0}
    finish: dict = {}

    def deps_of(a):
        if a.kind == "F":
            return [(a.stage - 1, "F", a.mb)] if a.stage > 0 else []
        if a.kind == "W":
            return [(a.stage, "B", a.mb)]
        return [(a.stage, "F", a.mb)] + ([(a.stage + 1, "B", a.mb)] if a.stage < num_stages - 1 else [])

    pos, free = [0] * len(ranks), [0.0] * len(ranks)
    progressed = True
    while progressed:
        progressed = False
        for r, acts in enumerate(ranks):
            while pos[r] < len(acts):
                parts = acts[pos[r]].parts()
                deps = [d for a in parts for d in deps_of(a)]
                if any(d not in finish for d in deps):
                    break
                work = sum(cost[a.kind] for a in parts) * (1.0 - pair_credit if len(parts) > 1 else 1.0)
                end = max([free[r]] + [finish[d] for d in deps]) + work
                for a in parts:
                    finish[(a.stage, "B" if a.kind == "I" else a.kind, a.mb)] = end
                free[r] = end
                pos[r] += 1
                progressed = True
    total = max(free)
    busy = max(sum(cost[b.kind] for a in acts for b in a.parts()) for acts in ranks)
    return total, 1.0 - busy / total if total else 0.0


# ------------------------------------------------------------------------------------ runtime
_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64]


def _micro_batch_of(v, n: int, m: int, bs: int | None):
    """Micro-batch ``m`` of ``n`` of a keyword argument: tensors whose leading dimension is the batch are cut, containers
    (dicts, mask records) are walked, everything else is passed whole."""
    import dataclasses

    if n <= 1 or bs is None:
        return v
    if torch.is_tensor(v):
        return torch.tensor_split(v, n, dim=0)[m] if v.dim() > 0 and v.shape[0] == bs else v
    if isinstance(v, dict):
        return {k: _micro_batch_of(x, n, m, bs) for k, x in v.items()}
    if dataclasses.is_dataclass(v) and not isinstance(v, type):
        changes = {}
        for f in dataclasses.fields(v):
            x = getattr(v, f.name)
            if torch.is_tensor(x) and x.dim() > 1 and x.shape[0] == bs:
                changes[f.name] = torch.tensor_split(x, n, dim=0)[m]
        if changes:
            # packed boundaries describe the whole batch: the per-row ids carry the same information
            for name in ("cu_seqlens", "max_seqlen"):
                if hasattr(v, name) and name not in changes:
                    changes[name] = None
            return dataclasses.replace(v, **changes)
    return v


def _batch_size_hint(kwargs) -> int | None:
    import dataclasses

    for v in kwargs.values():
        for x in (v.values() if isinstance(v, dict) else (v,)):
            if dataclasses.is_dataclass(x) and not isinstance(x, type):
                for f in dataclasses.fields(x):
                    t = getattr(x, f.name)
                    if torch.is_tensor(t) and t.dim() > 1:
                        return t.shape[0]
    return None


class PipelineSchedule:
    """Executes one rank's action list. Messages between two ranks are FIFO and untagged (NCCL), so
    the receiver consumes them in the *sender's* order, which it derives from the global schedule,
    and parks early arrivals until the action that needs them runs."""

    def __init__(self, *, stages: dict[int, nn.Module], all_actions: list[list[Action]], pp_group, pp_rank: int, pp: int,
                 num_stages: int, n_microbatches: int, loss_fn, style: str, device):
        self.stages, self.all_actions = stages, all_actions
        self.group, self.rank, self.pp = pp_group, pp_rank, pp
        self.num_stages, self.n_mb, self.loss_fn, self.style, self.device = num_stages, n_microbatches, loss_fn, style, device
        self._meta: dict = {}
        self.has_first = 0 in stages
        self.has_last = (num_stages - 1) in stages

    def _rank_of(self, stage: int) -> int:
        return stage_to_rank(stage, self.pp, self.num_stages, self.style)

    def _inbound_orders(self, actions_per_rank) -> dict[int, list]:
        """For every peer: the (kind, dst_stage, mb) messages it sends to this rank, in its order."""
        orders: dict[int, list] = {}
        for r, acts in enumerate(actions_per_rank):
            if r == self.rank:
                continue
            seq = []
            for a in (b for a0 in acts for b in a0.parts()):
                if a.kind == "F" and a.stage < self.num_stages - 1 and self._rank_of(a.stage + 1) == self.rank:
                    seq.append(("act", a.stage + 1, a.mb))
                if a.kind in ("B", "I") and a.stage > 0 and self._rank_of(a.stage - 1) == self.rank:
                    seq.append(("grad", a.stage - 1, a.mb))
            orders[r] = seq
        return orders

    # ---- point to point -------------------------------------------------------------------------
    def _send(self, t: torch.Tensor, kind: str, dst_stage: int, pending: list):
        dst = dist.get_global_rank(self.group, self._rank_of(dst_stage))
        key = ("sent", kind, dst_stage)
        if key not in self._meta:
            meta = torch.zeros(8, dtype=torch.int64)
            meta[0] = t.dim()
            meta[1 : 1 + t.dim()] = torch.tensor(list(t.shape))
            meta[7] = _DTYPES.index(t.dtype)
            dist.send(meta.to(self.device), dst, group=self.group)
            self._meta[key] = True
        t = t.contiguous()
        pending.append((dist.isend(t, dst, group=self.group), t))

    def _recv(self, kind: str, dst_stage: int, mb: int, src_stage: int) -> torch.Tensor:
        peer = self._rank_of(src_stage)
        want = (kind, dst_stage, mb)
        box = self._inbox.setdefault(peer, {})
        src = dist.get_global_rank(self.group, peer)
        while want not in box:
            cur = self._cursor.get(peer, 0)
            order = self._orders[peer]
            assert cur < len(order), f"pipeline rank {self.rank}: {want} never sent by rank {peer}"
            k, st, m = order[cur]
            self._cursor[peer] = cur + 1
            mkey = ("recv", k, st)
            if mkey not in self._meta:
                meta = torch.zeros(8, dtype=torch.int64, device=self.device)
                dist.recv(meta, src, group=self.group)
                meta = meta.cpu()
                nd = int(meta[0])
                self._meta[mkey] = (tuple(int(v) for v in meta[1 : 1 + nd]), _DTYPES[int(meta[7])])
            shape, dtype = self._meta[mkey]
            buf = torch.empty(shape, dtype=dtype, device=self.device)
            dist.recv(buf, src, group=self.group)
            box[(k, st, m)] = buf
        return box.pop(want)

    # ---- one optimizer step worth of micro-batches --------------------------------------------------
    def _run(self, actions_per_rank, args, kwargs, target, losses, loss_scale, train: bool):
        n = self.n_mb
        self._orders = self._inbound_orders(actions_per_rank)
        self._cursor, self._inbox, self._local_grads = {}, {}, {}
        inputs_mb = None
        bs = None
        if self.has_first:
            assert args, "the first pipeline stage needs the model input"
            bs = args[0].shape[0]
            inputs_mb = list(torch.tensor_split(args[0], n, dim=0)) if n > 1 else [args[0]]
        elif target is not None:
            bs = target.shape[0]
        if bs is None:
            bs = _batch_size_hint(kwargs)            # a middle stage sees neither the tokens nor the labels
        kw_mb = [{k: _micro_batch_of(v, n, m, bs) for k, v in kwargs.items()} for m in range(n)]
        target_mb = None
        if target is not None:
            target_mb = list(torch.tensor_split(target, n, dim=0)) if n > 1 else [target]
        saved: dict = {}
        pending: list = []
        parked: dict = {}                                # (stage, mb) -> weight-gradient closures of its "I" action
        last_stage = self.num_stages - 1

        def forward_input(a):
            if a.stage == 0:
                return inputs_mb[a.mb]
            if (a.stage - 1) in self.stages:
                return saved[(a.stage - 1, a.mb)][1].detach()
            return self._recv("act", a.stage, a.mb, a.stage - 1)

        def forward_compute(a, x):
            if a.stage != 0 and train:
                x.requires_grad_(True)
            with torch.set_grad_enabled(train):
                out = self.stages[a.stage](x, **kw_mb[a.mb])
                if a.stage == last_stage:
                    loss_sum = self.loss_fn(out, target_mb[a.mb])
                    val = loss_sum * loss_scale if loss_scale is not None else loss_sum
                    if losses is not None:
                        losses.append(val.detach().reshape(()))
                    out = val
            saved[(a.stage, a.mb)] = (x, out)
            return out

        def forward_send(a, out):
            if a.stage != last_stage and (a.stage + 1) not in self.stages:
                self._send(out.detach(), "act", a.stage + 1, pending)

        def backward_input(a):
            if a.stage == last_stage:
                return None
            if (a.stage + 1) in self.stages:
                return self._local_grads.pop((a.stage, a.mb))
            return self._recv("grad", a.stage, a.mb, a.stage + 1)

        def backward_compute(a, g):
            x, out = saved.pop((a.stage, a.mb))
            if a.kind == "I":
                with WeightGradStore.collect() as queue:
                    torch.autograd.backward(out, g)
                parked[(a.stage, a.mb)] = queue
            else:
                torch.autograd.backward(out, g)
            return x.grad if a.stage != 0 else None

        def backward_send(a, gx):
            if a.stage == 0:
                return
            if (a.stage - 1) in self.stages:
                self._local_grads[(a.stage - 1, a.mb)] = gx
            else:
                self._send(gx, "grad", a.stage - 1, pending)

        for a in actions_per_rank[self.rank]:
            if a.kind == "W":
                WeightGradStore.run(parked.pop((a.stage, a.mb)))
            elif a.kind == "F":
                forward_send(a, forward_compute(a, forward_input(a)))
            elif a.kind == "O":
                # a forward and a backward of different micro-batches in one slot: inputs first, then the two computations
                # taking turns at their expert-parallel exchanges, then the outputs in the order the peers expect
                from .overlap import run_overlapped

                f, b = a.parts()
                x, g = forward_input(f), backward_input(b)
                out, gx = run_overlapped(lambda: forward_compute(f, x), lambda: backward_compute(b, g))
                forward_send(f, out)
                backward_send(b, gx)
            else:
                backward_send(a, backward_compute(a, backward_input(a)))
            pending = [(w, t) for (w, t) in pending if not w.is_completed()]
        for w, _ in pending:
            w.wait()
        assert not parked, f"weight-gradient steps never ran for {sorted(parked)}"

    def step(self, *args, target=None, losses=None, loss_scale=None, return_outputs: bool = False, **kwargs):
        self._run(self.all_actions, args, kwargs, target, losses, loss_scale, train=True)

    def eval(self, *args, target=None, losses=None, **kwargs):
        fwd_only = [[b for a in acts for b in a.parts() if b.kind == "F"] for acts in self.all_actions]
        with torch.no_grad():
            self._run(fwd_only, args, kwargs, target, losses, None, train=False)


# ------------------------------------------------------------------------------------ entry point
def pipeline_llm(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config, ac_config,
                 dump_folder: str, device, model_config, parallelize_fn, loss_fn):
    pp_mesh = parallel_dims.get_mesh("pp")
    pp, pp_rank = pp_mesh.size(), pp_mesh.get_local_rank()
    schedule = parallelism.pipeline_parallel_schedule
    csv_path = parallelism.pipeline_parallel_schedule_csv
    if schedule not in SCHEDULES and not csv_path:
        raise ValueError(f"Unknown pipeline schedule {schedule}; supported: {sorted(SCHEDULES)}")
    single = schedule in SINGLE_STAGE
    if not hasattr(model_config, "n_layers"):
        raise ValueError("Model does not have n_layers attribute.")
    num_layers = model_config.n_layers
    in_w = parallelism.pipeline_parallel_first_stage_less_layers
    out_w = parallelism.pipeline_parallel_last_stage_less_layers
    per_stage = parallelism.pipeline_parallel_layers_per_stage
    fqns = parallelism.module_fqns_per_model_part
    if fqns is None:
        if per_stage is not None:
            num_stages = math.ceil((num_layers + in_w + out_w) / per_stage)
            if num_stages % pp != 0:
                raise ValueError(
                    f"Number of virtual stages ({num_stages}) must be divisible by pipeline parallel size ({pp}). "
                    f"Model has {num_layers} layers with pipeline_parallel_layers_per_stage={per_stage}."
                )
            spr = num_stages // pp
            if single and spr != 1:
                raise ValueError(f"Single stage schedule requires exactly 1 stage per rank, but got {spr} stages per rank.")
            if not single and spr < 2:
                raise ValueError(f"Multi-stage schedule requires at least 2 stages per rank, but got {spr} stages per rank.")
        else:
            num_stages = pp * (1 if single else 2)
        fqns = generate_llm_fqn_per_model_part(num_stages, num_layers, in_w, out_w)
    num_stages = len(fqns)
    idx, parts, style = pipeline_module_split(model, pp_rank, pp, schedule, fqns)
    for i, m in enumerate(parts):
        parts[i] = parallelize_fn(
            m, parallel_dims=parallel_dims, training=training, model_converters=model_converters, parallelism=parallelism,
            compile_config=compile_config, ac_config=ac_config, dump_folder=dump_folder,
        )
    mbs = parallelism.pipeline_parallel_microbatch_size
    if training.local_batch_size % mbs != 0:
        raise ValueError(f"Batch size {training.local_batch_size} must be divisible by microbatch_size {mbs}.")
    n_mb = training.local_batch_size // mbs
    if n_mb < num_stages:
        logger.warning(
            f"Number of microbatches ({n_mb}) is less than the total number of stages ({num_stages}) which may result in a bubble in the pipeline."
        )
    from .fsdp import fsdp_units

    # weight gradients of linear layers can be parked wherever the weight owns its .grad (pipeline-only, tensor parallel)
    # or comes from an FSDP / replicate unit, which then queues its gradient reduction behind the parked GEMMs
    can_split = True
    sharded = any(fsdp_units(m) for m in parts)
    if csv_path:
        all_actions = load_csv_actions(csv_path)
        assert len(all_actions) == pp, f"CSV schedule has {len(all_actions)} rows for {pp} pipeline ranks"
        if not can_split:
            all_actions = fuse_split_backward(all_actions)
    else:
        # DualPipeV with expert parallel: forward / backward neighbours share a slot so that the token exchanges of one hide
        # behind the compute of the other
        all_actions = build_actions(schedule, pp, num_stages, n_mb, style, split=can_split,
                                    overlap=bool(getattr(parallel_dims, "ep_enabled", False)))
    validate_actions(all_actions, pp, num_stages, n_mb, style)
    sched = PipelineSchedule(
        stages=dict(zip(idx, parts)), all_actions=all_actions, pp_group=pp_mesh.get_group(), pp_rank=pp_rank, pp=pp,
        num_stages=num_stages, n_microbatches=n_mb, loss_fn=loss_fn, style=style, device=device,
    )
    logger.info(f"Using pipeline schedule {schedule if not csv_path else csv_path} with {n_mb} microbatches and {num_stages} stages.")
    has_split = any(a.kind in ("I", "W") for acts in all_actions for a in acts)
    WeightGradStore.enabled = has_split
    n_pairs = sum(1 for acts in all_actions for a in acts if a.kind == "O")
    if n_pairs:
        logger.info(f"{n_pairs} pipeline slots run a forward and a backward of different micro-batches together")
    logger.info("Pipeline bubble estimate (forward 1, backward 2 units per stage and micro-batch): "
                f"{estimate_makespan(all_actions, num_stages)[1]:.1%} of the step")
    if has_split:
        logger.info("Pipeline backward steps are split: input gradients are sent on first, the weight gradients of the "
                    "linear layers run where the rank would wait"
                    + (" and end with the FSDP / replicate units' gradient reduction" if sharded else ""))
    return sched, parts, sched.has_first, sched.has_last

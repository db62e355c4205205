"""Asynchronous tensor parallel: the sequence all-gather fused into the GEMM that consumes it.

Reference behaviour (``enable_async_tensor_parallel``, torchtitan/distributed/tensor_parallel.py:202 -> the
symmetric-memory micro-pipeline of upstream PyTorch): decompose all-gather -> matmul into chunks so transfers hide
behind the math. Here it is one kernel (``tt_gemm_allgather_a`` in ``csrc/gemm.cu``): every rank keeps the gathered
activation buffer in its NVLink-mapped symmetric heap and writes its own sequence slice there; in the fused launch a few
CTAs pull the peers' slices panel by panel (128 rows) with plain peer loads while the other CTAs run the tcgen05 GEMM,
local panels first, each output tile waiting only for the panel it reads. The gathered activation stays in the local
buffer, so the other projections of the block (``w3`` next to ``w1``) read it without another collective.

Buffers are double-buffered per shape and versioned by a job-wide call counter; a rank overwrites a slice only after it
has seen the peers' flags of the following version, which they publish after their own fused kernel finished reading.

The mirror image closes a row-parallel layer (``w2``, ``wo``): ``tt_gemm_reduce_scatter`` computes the partial product of
this rank's K-shard and its epilogue stores each output tile, as bf16, straight into the staging slot of the rank that
owns those rows (peer stores over NVLink), remote-owned tiles first, and bumps the owner's counter for that tile with a
system-scope atomic; the tiles of this rank's own rows come last, and their epilogue waits for the peers' counters, adds
the staged partials to the fp32 accumulator in rank order and writes the final rows. Staging is double-buffered: a rank's call n+1 ends only after every peer contributed to
call n+1, which they do after their call n, so the buffer of call n is free again when call n+2 starts.

Backward reuses both kernels with the weight read as the [contraction, output] operand: the input gradient of a
column-parallel layer is a GEMM -> reduce-scatter, that of a row-parallel layer an all-gather -> GEMM whose gathered
output gradient also feeds the weight-gradient GEMM. Only the re-gather of the saved sequence shard for the weight
gradients of column-parallel layers is a plain collective.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from torchtitan_b200.ops import native
from torchtitan_b200.tools.logging import logger

from .nvlink_comm import _PP, SymmetricHeap, _stream, peer_memory_group_ok


class AsyncTP:
    COPY_CTAS = 8     # measured optimum on the isolated kernel at tp = 2: more copy CTAs take tensor-core SMs for no extra link throughput

    def __init__(self, tp_mesh, heap_bytes: int = 1 << 30):
        self.group = tp_mesh.get_group()
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.heap = SymmetricHeap(self.group, heap_bytes, self.device)
        self.world, self.rank = self.heap.world, self.heap.rank
        self.flag_off = self.heap.alloc_flag()
        self._flag_ptrs, self._flag_keep = self.heap.peer_ptrs(self.flag_off)
        self._bufs: dict[tuple[int, int], list] = {}
        self.version = 0
        self.panel_ready = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.fused_calls = 0
        self._rs_bufs: dict[tuple[int, int], list] = {}
        self.rs_calls = 0

    @classmethod
    def maybe_create(cls, tp_mesh):
        if not native.available() or not native.has("tt_gemm_allgather_a"):
            return None
        if not peer_memory_group_ok(tp_mesh.get_group()):
            return None
        return cls(tp_mesh)

    # ---- buffers --------------------------------------------------------------------------------------------
    def _buffers(self, rows: int, K: int):
        key = (rows, K)
        if key not in self._bufs:
            out = []
            for _ in range(2):
                off = self.heap.alloc(rows * K * 2, align=1024)
                ptrs, keep = self.heap.peer_ptrs(off)
                out.append((off, ptrs, keep, self.heap.local_tensor(off, rows * K, torch.bfloat16).view(rows, K)))
            self._bufs[key] = out
        return self._bufs[key]

    def supported(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        rows_local = x.numel() // x.shape[-1]
        return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] == 1
                and rows_local % 128 == 0 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
                and rows_local * self.world // 128 <= self.panel_ready.numel())

    def ag_linear(self, x: torch.Tensor, weight: torch.Tensor):
        """``x`` [1, S/tp, K] (this rank's sequence slice), ``weight`` [N, K] -> (gathered x [1, S, K], x_full @ weight^T)."""
        return _AgLinear.apply(x, weight, self)

    def _forward(self, x: torch.Tensor, weight: torch.Tensor, b_mn: bool = False):
        """Fused gather of ``x`` + GEMM with ``weight`` [N, K] (or stored [K, N] with ``b_mn``, as in the input-gradient
        GEMM of a row-parallel layer)."""
        L = native.lib()
        K = x.shape[-1]
        rows_local = x.numel() // K
        rows = rows_local * self.world
        N = weight.shape[1] if b_mn else weight.shape[0]
        self.version += 1
        off, ptrs, _keep, full = self._buffers(rows, K)[self.version % 2]
        full[self.rank * rows_local : (self.rank + 1) * rows_local].copy_(x.reshape(rows_local, K))
        native.check(L.tt_set_flag(self.heap.base + self.flag_off, self.version, _stream()), "tt_set_flag")
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        w = weight.contiguous()
        native.check(L.tt_gemm_allgather_a(ptrs, ctypes.cast(self._flag_ptrs, _PP), self.world, self.rank, self.version,
                                           w.data_ptr(), out.data_ptr(), rows, N, K, int(b_mn), w.stride(0), out.stride(0), 0,
                                           self.panel_ready.data_ptr(), self.version, self.COPY_CTAS, _stream()),
                     "tt_gemm_allgather_a")
        self.fused_calls += 1
        return full.view(1, rows, K), out.view(1, rows, N)

    # ---- GEMM -> reduce-scatter ----------------------------------------------------------------------------
    def _rs_buffers(self, rows: int, N: int):
        """Two (staging, counters) sets for outputs of ``rows`` x ``N``; each entry also counts its own calls."""
        key = (rows, N)
        if key not in self._rs_bufs:
            out = []
            panels = rows // self.world // 128
            for _ in range(2):
                soff = self.heap.alloc(rows * N * 2, align=1024)
                coff = self.heap.alloc(self.world * panels * ((N + 255) // 256) * 4, align=256)
                sp, sk = self.heap.peer_ptrs(soff)
                cp, ck = self.heap.peer_ptrs(coff)
                out.append({"stage": sp, "count": cp, "keep": (sk, ck), "calls": 0})
            self._rs_bufs[key] = out
        return self._rs_bufs[key]

    def rs_supported(self, h: torch.Tensor, weight: torch.Tensor) -> bool:
        rows = h.numel() // h.shape[-1]
        return (native.has("tt_gemm_reduce_scatter") and h.is_cuda and h.dtype == torch.bfloat16
                and weight.dtype == torch.bfloat16 and h.shape[0] == 1 and rows % (128 * self.world) == 0
                and h.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0)

    def linear_rs(self, h: torch.Tensor, weight: torch.Tensor):
        """``h`` [1, S, K/tp] (this rank's feature shard), ``weight`` [N, K/tp] -> this rank's sequence slice
        [1, S/tp, N] of ``sum over ranks (h @ weight^T)``."""
        return _LinearRs.apply(h, weight, self)

    def _forward_rs(self, h: torch.Tensor, weight: torch.Tensor, b_mn: bool = False):
        L = native.lib()
        K = h.shape[-1]
        rows = h.numel() // K
        N = weight.shape[1] if b_mn else weight.shape[0]
        h2 = h.reshape(rows, K)
        if h2.stride(-1) != 1 or h2.stride(0) % 8:
            h2 = h2.contiguous()
        w = weight.contiguous()
        self.rs_calls += 1
        buf = self._rs_buffers(rows, N)[self.rs_calls % 2]
        buf["calls"] += 1
        out = torch.empty(rows // self.world, N, dtype=torch.bfloat16, device=h.device)
        native.check(L.tt_gemm_reduce_scatter(h2.data_ptr(), w.data_ptr(), buf["stage"], ctypes.cast(buf["count"], _PP),
                                              out.data_ptr(), self.world, self.rank, rows, N, K, h2.stride(0), int(b_mn),
                                              w.stride(0), buf["calls"], 0, _stream()),
                     "tt_gemm_reduce_scatter")
        self.fused_calls += 1
        return out.view(1, rows // self.world, N)

    # ---- module hooks used by the tensor-parallel plan ---------------------------------------------------------
    def attach_ffn(self, ff) -> None:
        ff._async_tp = self

    def attach_attention(self, att) -> None:
        """Grouped-query attention without biases: ``wq`` gathers the sequence inside its GEMM, ``wk`` / ``wv`` read the
        gathered copy, ``wo`` reduce-scatters inside its GEMM. Other attention forms keep the collective path."""
        plain = all(hasattr(att, n) for n in ("wq", "wk", "wv", "wo")) and not hasattr(att, "wkv_b") and all(
            getattr(getattr(att, n), "bias", None) is None and getattr(getattr(att, n), "quant", None) is None
            for n in ("wq", "wk", "wv", "wo"))
        att._async_tp = self if plain else None

    def attention_supported(self, att, x_local: torch.Tensor) -> bool:
        if getattr(att, "_async_tp", None) is not self or not self.supported(x_local, att.wq.weight):
            return False
        rows = x_local.shape[1] * self.world
        return (native.has("tt_gemm_reduce_scatter") and rows % (128 * self.world) == 0
                and att.wo.weight.dtype == torch.bfloat16 and att.wo.weight.shape[0] % 8 == 0 and att.wo.weight.shape[1] % 8 == 0)

    def project(self, att, x_local):
        xg, q = self.ag_linear(x_local, att.wq.weight)
        k = _LinearOnGathered.apply(xg, x_local, att.wk.weight, self.group, self)
        v = _LinearOnGathered.apply(xg, x_local, att.wv.weight, self.group, self)
        return q, k, v

    def output(self, att, o):
        return self.linear_rs(o, att.wo.weight)


class _AgLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, atp: AsyncTP):
        xg, y = atp._forward(x, weight)
        ctx.save_for_backward(x, weight)
        ctx.atp = atp
        ctx.mark_non_differentiable(xg)
        # the gathered buffer is recycled two calls later: hand out a view for immediate consumers only
        return xg, y

    @staticmethod
    def backward(ctx, _gxg, gy):
        from .tp import all_gather_seq

        x, weight = ctx.saved_tensors
        atp = ctx.atp
        group, W = atp.group, atp.world
        gy2 = gy.reshape(-1, gy.shape[-1])
        gx = _input_grad_rs(atp, gy2, weight)
        gw = gy2.t() @ _regather(atp, x)
        return gx.view_as(x), gw, None


def _regather(atp: "AsyncTP", x: torch.Tensor) -> torch.Tensor:
    """The sequence-gathered copy of the saved shard ``x`` for a weight gradient. The projections that read the same
    input (``wq`` / ``wk`` / ``wv``, ``w1`` / ``w3``) run their backward one after another: the last gathered copy is kept
    and reused while the same tensor (same storage, same version) is asked for, so it is gathered once per group."""
    from .tp import all_gather_seq

    key = (x.data_ptr(), x._version, tuple(x.shape))
    hit = atp.__dict__.get("_regather_cache")
    if hit is not None and hit[0] == key:
        return hit[2]
    xg = all_gather_seq(x.detach(), atp.group).reshape(-1, x.shape[-1])
    # the entry keeps ``x`` itself: while it is held its memory cannot be handed to another tensor, so an equal address
    # (with an equal version) can only be the same activation
    atp.__dict__["_regather_cache"] = (key, x, xg)
    return xg


def _input_grad_rs(atp: "AsyncTP", gy2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``reduce_scatter_rows(gy2 @ weight)`` for a column-parallel layer's input gradient: the fused GEMM ->
    reduce-scatter when the shapes allow (``weight`` [N, K] is read as the [contraction, output] operand), else the
    collective."""
    W = atp.world
    gy2 = gy2 if gy2.is_contiguous() else gy2.contiguous()
    rows = gy2.shape[0]
    if (native.has("tt_gemm_reduce_scatter") and gy2.is_cuda and gy2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and rows % (128 * W) == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0):
        return atp._forward_rs(gy2.view(1, rows, -1), weight, b_mn=True).view(rows // W, weight.shape[1])
    gx_full = gy2 @ weight
    gx = torch.empty(rows // W, gx_full.shape[1], dtype=gx_full.dtype, device=gx_full.device)
    dist.reduce_scatter_tensor(gx, gx_full.contiguous(), group=atp.group)
    return gx


class _LinearRs(torch.autograd.Function):
    """Row-parallel linear closed by the fused reduce-scatter; backward gathers the output gradient (collective)."""

    @staticmethod
    def forward(ctx, h, weight, atp: AsyncTP):
        ctx.save_for_backward(h, weight)
        ctx.atp = atp
        return atp._forward_rs(h, weight)

    @staticmethod
    def backward(ctx, gy):
        from .tp import all_gather_seq

        h, weight = ctx.saved_tensors
        atp = ctx.atp
        gy = gy.contiguous()
        if atp.supported(gy, weight):
            # all-gather of the output gradient fused into the input-gradient GEMM; the gathered copy feeds the weight gradient
            g_full, gh = atp._forward(gy, weight, b_mn=True)
            g_full = g_full.reshape(-1, gy.shape[-1])
            gw = g_full.t() @ h.reshape(-1, h.shape[-1])
            return gh.view_as(h), gw, None
        g_full = all_gather_seq(gy, atp.group).reshape(-1, gy.shape[-1])                       # [S, N]
        gh = (g_full @ weight).view_as(h)
        gw = g_full.t() @ h.reshape(-1, h.shape[-1])
        return gh, gw, None


def fused_ffn_forward(ff, x_local, group):
    """SwiGLU feed-forward under sequence parallel with the all-gather fused into ``w1``; returns the partial-sum output
    [1, S, D] and False (the caller reduce-scatters it), or -- when the fused GEMM -> reduce-scatter applies to ``w2`` --
    this rank's sequence slice [1, S/tp, D] and True."""
    from torchtitan_b200 import ops

    atp: AsyncTP = ff._async_tp
    xg, h1 = atp.ag_linear(x_local, ff.w1.weight)
    # w3 must use xg before the buffer is recycled; it is consumed right here. For backward it re-gathers (collective).
    h3 = _LinearOnGathered.apply(xg, x_local, ff.w3.weight, group, atp)
    h = ops.swiglu(h1, h3)
    if getattr(ff.w2, "bias", None) is None and getattr(ff.w2, "quant", None) is None and atp.rs_supported(h, ff.w2.weight):
        return atp.linear_rs(h, ff.w2.weight), True
    return ff.w2(h), False


class _LinearOnGathered(torch.autograd.Function):
    """``xg @ w^T`` where ``xg`` is a transient gathered copy of the sequence-sharded ``x``: saves only the shard."""

    @staticmethod
    def forward(ctx, xg, x_local, weight, group, atp=None):
        from torchtitan_b200 import ops

        ctx.save_for_backward(x_local, weight)
        ctx.group = group
        ctx.atp = atp
        with torch.no_grad():
            return ops.linear(xg, weight, None)

    @staticmethod
    def backward(ctx, gy):
        from .tp import all_gather_seq

        x, weight = ctx.saved_tensors
        W = dist.get_world_size(ctx.group)
        gy2 = gy.reshape(-1, gy.shape[-1])
        if ctx.atp is not None:
            gx = _input_grad_rs(ctx.atp, gy2, weight)
            return None, gx.view_as(x), gy2.t() @ _regather(ctx.atp, x), None, None
        else:
            gx_full = gy2 @ weight
            gx = torch.empty(gx_full.shape[0] // W, gx_full.shape[1], dtype=gx_full.dtype, device=gx_full.device)
            dist.reduce_scatter_tensor(gx, gx_full.contiguous(), group=ctx.group)
        xg = all_gather_seq(x.detach(), ctx.group).reshape(-1, x.shape[-1])
        return None, gx.view_as(x), gy2.t() @ xg, None, None

"""Expert-parallel dispatch / combine over NVLink peer memory (``csrc/ep.cu``): permutation and all-to-all in one kernel,
counts exchanged through peer memory, group offsets kept on the device -- no collective library call and no device-to-host
read on the path. Drop-in for :class:`parallel.ep.AllToAllDispatcher` (same ``dispatch`` / ``combine`` contract).

The receive buffer has a fixed capacity (plus alignment padding). Two modes:

* default (``capacity_factor=None``): lossless. The buffer holds three times the rows a rank sends; after the counts are
  exchanged every rank reads the (identical) count table on the host, and when any rank's experts would receive more
  than the buffer holds, this call goes through the all-to-all dispatcher instead. One small device-to-host read per
  dispatch, no token is ever dropped (what the reference's DeepEP backend guarantees by default);
* ``hybridep_non_blocking_expert_capacity_factor`` set: no host read at all; rows beyond ``factor x`` the rows a rank sends
  are dropped and reported through ``native.kernel_errors()`` (the reference's non-blocking HybridEP mode).

Received rows are copied out of the symmetric buffer (which is recycled two calls later) into an ordinary tensor, with the
padding rows zeroed in the same pass.
Parity: the DeepEP / HybridEP backends of the reference (torchtitan/distributed/deepep, hybridep: NVLink buffers, fused
permute, optional fixed-capacity non-blocking mode), without the external library."""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from torchtitan_b200.ops import native

from .nvlink_comm import _PP, SymmetricHeap, _stream, peer_memory_group_ok


def copy_rows_where(rows, keep):
    from torchtitan_b200.ops.cuda_ops import copy_rows_where as f

    return f(rows, keep)


def sum_copies(rows, pos, num_tokens, top_k):
    from torchtitan_b200.ops.cuda_ops import sum_copies as f

    return f(rows, pos, num_tokens, top_k)


def inverse_positions(order):
    from torchtitan_b200.ops.cuda_ops import inverse_positions as f

    return f(order)

_I32 = torch.int32


class _Shared:
    """Buffers and call counters shared by all MoE layers of one expert-parallel group with the same (rows, width)."""

    def __init__(self, heap: SymmetricHeap, n: int, D: int, E: int, cap: int):
        self.heap, self.n, self.D, self.E, self.cap = heap, n, D, E, cap
        W = heap.world
        self.recv, self.ret, self.table, self.flags, self.arrive = [], [], [], [], {"fwd": [], "rev": []}
        for _ in range(2):
            self.recv.append(self._buf(cap * D * 2, cap * D, torch.bfloat16, (cap, D)))
            self.ret.append(self._buf(n * D * 2, n * D, torch.bfloat16, (n, D)))
            self.table.append(self._buf(W * E * 4, W * E, _I32, (W, E)))
            self.flags.append(self._buf(W * 4, W, _I32, (W,)))
            for d in ("fwd", "rev"):
                self.arrive[d].append(self._buf(4, 1, _I32, (1,)))
        self.dispatch_calls = 0
        self.dir_calls = {"fwd": 0, "rev": 0}
        self.ctas = native.lib().tt_ep_push_ctas()

    def _buf(self, nbytes, numel, dtype, shape):
        off = self.heap.alloc(nbytes, align=1024)
        ptrs, keep = self.heap.peer_ptrs(off)
        return {"local": self.heap.local_tensor(off, numel, dtype).view(shape), "peers": ptrs, "keep": keep,
                "ptr": self.heap.base + off}


class _Exchange(torch.autograd.Function):
    """``direction == "fwd"``: this rank's rows (optionally gathered through ``in_index``) -> the owners' expert-grouped
    buffers, returns this rank's received rows [cap, D]; ``"rev"``: received-layout rows -> the sources' sorted order,
    returns [n, D]. Backward is the opposite direction."""

    @staticmethod
    def forward(ctx, rows, in_index, maps, sh: _Shared, direction: str, pos=None, top_k: int = 0):
        ctx.maps, ctx.sh, ctx.direction = maps, sh, direction
        ctx.in_index, ctx.in_rows, ctx.pos, ctx.top_k = in_index, rows.shape[0], pos, top_k
        return _exchange(rows, in_index, maps, sh, direction)

    @staticmethod
    def backward(ctx, g):
        sh, maps = ctx.sh, ctx.maps
        back = "rev" if ctx.direction == "fwd" else "fwd"
        out = _exchange(g.contiguous(), None, maps, sh, back)
        if ctx.direction == "fwd" and ctx.in_index is not None:
            # rows were gathered through in_index: add the gradients of the copies of each source row
            if ctx.pos is not None and out.dtype == torch.bfloat16:
                return sum_copies(out, ctx.pos, ctx.in_rows, ctx.top_k), None, None, None, None, None, None
            gx = g.new_zeros(ctx.in_rows, g.shape[-1])
            gx.index_add_(0, ctx.in_index.long(), out)
            return gx, None, None, None, None, None, None
        return out, None, None, None, None, None, None


class _ExchangeScores(torch.autograd.Function):
    """One fp32 value per sorted row -> one per received row (and back for the gradient). A value rides in the first four
    bytes of a 16-byte row, which the row kernels move as eight bf16 elements without looking at them."""

    @staticmethod
    def _pack(v):
        buf = torch.zeros(v.shape[0], 4, dtype=torch.float32, device=v.device)
        buf[:, 0] = v
        return buf.view(torch.bfloat16)                                   # [rows, 8]

    @staticmethod
    def _unpack(rows):
        return rows.contiguous().view(torch.float32)[:, 0].clone()

    @staticmethod
    def forward(ctx, scores, maps, sh8):
        ctx.maps, ctx.sh8 = maps, sh8
        return _ExchangeScores._unpack(_exchange(_ExchangeScores._pack(scores), None, maps, sh8, "fwd"))

    @staticmethod
    def backward(ctx, g):
        back = _exchange(_ExchangeScores._pack(g.contiguous().float()), None, ctx.maps, ctx.sh8, "rev")
        return _ExchangeScores._unpack(back), None, None


def _exchange(rows, in_index, maps, sh: _Shared, direction: str):
    L = native.lib()
    W = sh.heap.world
    sh.dir_calls[direction] += 1
    par = sh.dir_calls[direction] % 2
    per_parity_calls = (sh.dir_calls[direction] + 1) // 2 if par else sh.dir_calls[direction] // 2   # calls on this buffer
    arrive = sh.arrive[direction][par]
    if direction == "fwd":
        n_in = maps["n"] if in_index is not None else rows.shape[0]
        native.check(L.tt_ep_push(rows.data_ptr(), in_index.data_ptr() if in_index is not None else None, n_in,
                                  maps["dst_rank"].data_ptr(), maps["dst_row"].data_ptr(), sh.recv[par]["peers"],
                                  arrive["peers"], W, sh.D, sh.cap, _stream()), "tt_ep_push")
        native.check(L.tt_ep_wait(arrive["ptr"], per_parity_calls * W * sh.ctas, _stream()), "tt_ep_wait")
        # copied out of the symmetric buffer (the exchange after next overwrites it), padding rows zeroed, in one pass
        return copy_rows_where(sh.recv[par]["local"], maps["rev_rank"] >= 0)
    native.check(L.tt_ep_push(rows.data_ptr(), None, sh.cap, maps["rev_rank"].data_ptr(), maps["rev_row"].data_ptr(),
                              sh.ret[par]["peers"], arrive["peers"], W, sh.D, sh.n, _stream()), "tt_ep_push")
    native.check(L.tt_ep_wait(arrive["ptr"], per_parity_calls * W * sh.ctas, _stream()), "tt_ep_wait")
    # rows that did not fit a receive buffer come back as zeros; copied out of the symmetric buffer in the same pass
    return copy_rows_where(sh.ret[par]["local"], maps["dst_rank"] >= 0)


class NvlinkDispatcher:
    _heaps: dict = {}
    _shared: dict = {}

    def __init__(self, ep_mesh, num_experts: int, alignment: int = 64, capacity_factor: float | None = None,
                 heap_bytes: int = 3 << 30):
        self.group = ep_mesh.get_group()
        self.ep, self.rank = ep_mesh.size(), ep_mesh.get_local_rank()
        assert num_experts % self.ep == 0, f"ep ({self.ep}) must divide num_experts ({num_experts})"
        self.num_experts, self.local_experts = num_experts, num_experts // self.ep
        self.alignment = alignment
        self.lossless = capacity_factor is None
        # lossless mode: room for three times the average load before a call has to take the collective path (with random
        # weights single ranks see more than twice the average in the first steps)
        self.capacity_factor = capacity_factor if capacity_factor is not None else 3.0
        self.heap_bytes = heap_bytes
        self.fallback_calls = 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._mesh, self._fallback = ep_mesh, None

    @classmethod
    def available(cls, ep_mesh) -> bool:
        if not (torch.cuda.is_available() and native.available() and native.has("tt_ep_push")):
            return False
        return peer_memory_group_ok(ep_mesh.get_group())

    def _state(self, n: int, D: int) -> _Shared:
        gid = id(self.group)
        if gid not in NvlinkDispatcher._heaps:
            NvlinkDispatcher._heaps[gid] = SymmetricHeap(self.group, self.heap_bytes, self.device)
        key = (gid, n, D, self.num_experts, self.capacity_factor)
        if key not in NvlinkDispatcher._shared:
            cap = int(n * self.capacity_factor) + self.local_experts * self.alignment
            cap = (cap + self.alignment - 1) // self.alignment * self.alignment
            NvlinkDispatcher._shared[key] = _Shared(NvlinkDispatcher._heaps[gid], n, D, self.num_experts, cap)
            dist.barrier(group=self.group)
        return NvlinkDispatcher._shared[key]

    def _collective(self):
        if self._fallback is None:
            from .ep import AllToAllDispatcher

            self._fallback = AllToAllDispatcher(self._mesh, self.num_experts, alignment=self.alignment)
        return self._fallback

    def _would_overflow(self, table: torch.Tensor, cap: int) -> bool:
        """``table`` [W, E]: rows every rank sends to every expert (complete once the map kernel ran, which precedes this
        read on the stream). True when some rank's padded expert groups exceed the receive capacity."""
        from torch.utils._python_dispatch import _disable_current_modes

        # the one host read of the lossless mode. Done outside any dispatch mode: activation checkpointing would
        # otherwise record this copy in its per-op cache, and the replay in backward must read its own table
        with _disable_current_modes():
            per_expert = table.sum(0).cpu().view(self.ep, self.local_experts)
        padded = (per_expert + self.alignment - 1) // self.alignment * self.alignment
        return bool((padded.sum(1) > cap).any())

    def dispatch(self, x, order, counts, top_k: int):
        if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
            # the peer-memory kernels move bf16 rows of a multiple of 8 elements: anything else takes the collectives
            rows, sizes, ctx = self._collective().dispatch(x, order, counts, top_k)
            ctx["fallback"] = True
            return rows, sizes, ctx
        L = native.lib()
        n, D = order.numel(), x.shape[-1]
        sh = self._state(n, D)
        sh.dispatch_calls += 1
        par = sh.dispatch_calls % 2
        version = (sh.dispatch_calls + 1) // 2 if par else sh.dispatch_calls // 2      # dispatches on this count table
        W, E, dev = self.ep, self.num_experts, x.device
        c64 = counts.to(torch.int64).contiguous()
        native.check(L.tt_ep_publish_counts(c64.data_ptr(), sh.table[par]["peers"], sh.flags[par]["peers"], W, self.rank, E,
                                            version, _stream()), "tt_ep_publish_counts")
        maps = {"n": n, "dst_rank": torch.empty(n, dtype=_I32, device=dev), "dst_row": torch.empty(n, dtype=_I32, device=dev),
                "rev_rank": torch.empty(sh.cap, dtype=_I32, device=dev), "rev_row": torch.empty(sh.cap, dtype=_I32, device=dev),
                "offs": torch.empty(self.local_experts, dtype=_I32, device=dev), "info": torch.empty(2, dtype=_I32, device=dev)}
        native.check(L.tt_ep_build_maps_opt(sh.table[par]["ptr"], sh.flags[par]["ptr"], W, self.rank, E, self.alignment, n, sh.cap,
                                            version, maps["dst_rank"].data_ptr(),
                                            maps["dst_row"].data_ptr(), maps["rev_rank"].data_ptr(), maps["rev_row"].data_ptr(),
                                            maps["offs"].data_ptr(), maps["info"].data_ptr(), None, D, int(not self.lossless),
                                            _stream()), "tt_ep_build_maps")
        if self.lossless and self._would_overflow(sh.table[par]["local"], sh.cap):
            # every rank sees the same table, so all of them take the collective path for this call
            self.fallback_calls += 1
            rows, sizes, ctx = self._collective().dispatch(x, order, counts, top_k)
            ctx["fallback"] = True
            return rows, sizes, ctx
        src_index = (order // top_k).to(_I32).contiguous()
        recv = _Exchange.apply(x.contiguous(), src_index, maps, sh, "fwd", inverse_positions(order), top_k)
        offs = maps["offs"].to(torch.int64)
        sizes = offs - torch.cat((offs.new_zeros(1), offs[:-1]))
        sizes._tt_aligned = self.alignment
        return recv, sizes, {"maps": maps, "sh": sh}

    def scale_rows(self, rows, scores_sorted, ctx):
        """Routing scores applied before the experts: the fp32 scores travel through the same exchange as 16-byte rows."""
        if ctx.get("fallback"):
            return self._fallback.scale_rows(rows, scores_sorted, ctx)
        sh8 = self._state(ctx["maps"]["n"], 8)
        sc = _ExchangeScores.apply(scores_sorted.reshape(-1).float(), ctx["maps"], sh8)       # [cap] fp32, 0 on padding
        from torchtitan_b200.ops.cuda_ops import scale_rows

        return scale_rows(rows, sc)

    def combine(self, y, ctx):
        if ctx.get("fallback"):
            return self._fallback.combine(y, ctx)
        return _Exchange.apply(y.contiguous(), None, ctx["maps"], ctx["sh"], "rev")

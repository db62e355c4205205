"""Context parallelism (ring attention with causal load balancing).

Data path as in torchtitan/distributed/context_parallel.py:27-246 and torchtitan/trainer.py:614-622:
the trainer builds ``positions = arange(S)`` and shards inputs, labels, positions (and per-token
document ids) over the ``cp`` mesh; with the ``headtail`` balancer the sequence is cut into ``2*cp``
chunks and rank ``r`` owns chunks ``r`` and ``2*cp-1-r``, so every rank does the same amount of
causal work; RoPE is indexed by the explicit positions. Parameters are FSDP-sharded over
``dp_shard * cp`` and losses / gradient norms reduce over the ``loss`` mesh.

The attention itself (``RingAttention``) supports both rotate methods of
``parallelism.context_parallel_rotate_method`` (a dead option in the reference, real here):

* ``allgather``: K and V shards are gathered once; each local query chunk then attends its whole
  causal prefix in a single kernel call (the kernel handles ``Sq != Sk`` with a causal offset), so no
  partial results have to be merged. Backward reduce-scatters dK/dV to their owners. Document masks, sliding windows
  and attention sinks are served by this method (the per-token document ids are gathered alongside).
* ``alltoall``: K/V blocks travel around the ring in ``cp-1`` point-to-point steps; partial outputs are
  merged with their log-sum-exp in fp32; backward runs the ring again with the final (merged)
  statistics, dK/dV travelling with their block.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from torchtitan_b200 import ops
from torchtitan_b200.tools.logging import logger

__all__ = ["apply_cp_to_attention_module", "prepare_context_parallel_input", "cp_shard", "RingAttention",
           "headtail_indices"]


# ------------------------------------------------------------------------------------ sharding
def headtail_indices(seq_len: int, cp: int, rank: int, balanced: bool = True) -> torch.Tensor:
    """Global positions owned by ``rank`` (ascending)."""
    if not balanced:
        c = seq_len // cp
        return torch.arange(rank * c, (rank + 1) * c)
    assert seq_len % (2 * cp) == 0, f"sequence length {seq_len} must be divisible by 2*cp={2 * cp}"
    c = seq_len // (2 * cp)
    a, b = rank, 2 * cp - 1 - rank
    return torch.cat((torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)))


def cp_shard(cp_mesh, tensors, seq_dims, load_balancer: str | None = "headtail"):
    cp, r = cp_mesh.size(), cp_mesh.get_local_rank()
    out = []
    for t, d in zip(tensors, seq_dims):
        idx = headtail_indices(t.shape[d], cp, r, balanced=load_balancer is not None).to(t.device)
        out.append(t.index_select(d, idx))
    return out


def prepare_context_parallel_input(inputs, labels, extra_kwargs, cp_mesh, device, load_balancer: str | None = "headtail"):
    S = inputs.shape[1]
    positions = torch.arange(S, dtype=torch.int32, device=inputs.device).unsqueeze(0)
    inputs, labels, positions = cp_shard(cp_mesh, (inputs, labels, positions), (1, 1, 1), load_balancer)
    extra_kwargs = dict(extra_kwargs)
    extra_kwargs["positions"] = positions.to(torch.int64)
    masks = extra_kwargs.get("attention_masks")
    if masks is not None and getattr(masks, "doc_ids", None) is not None:
        import dataclasses

        (doc,) = cp_shard(cp_mesh, (masks.doc_ids,), (1,), load_balancer)
        extra_kwargs["attention_masks"] = dataclasses.replace(masks, doc_ids=doc, cu_seqlens=None)
        extra_kwargs["attention_masks"].doc_ids_full = masks.doc_ids
    return inputs, labels, extra_kwargs


# ------------------------------------------------------------------------------------ merge helper
def _merge(out_a, lse_a, out_b, lse_b):
    """Combine two partial attention results over disjoint key sets (fp32)."""
    if out_a is None:
        return out_b.float(), lse_b
    m = torch.maximum(lse_a, lse_b)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    wa, wb = torch.exp(lse_a - m), torch.exp(lse_b - m)
    denom = wa + wb
    lse = m + torch.log(denom)
    wa = (wa / denom).transpose(1, 2).unsqueeze(-1)  # [B,S,H,1]
    wb = (wb / denom).transpose(1, 2).unsqueeze(-1)
    return out_a * wa + out_b.float() * wb, lse


class _AllGatherKV(torch.autograd.Function):
    """Gather sequence chunks of K or V from all cp ranks into global chunk order; backward =
    reduce-scatter of the gradient to the owners."""

    @staticmethod
    def forward(ctx, x, group, balanced):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        ctx.group, ctx.balanced = group, balanced
        parts = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(parts, x.contiguous(), group=group)
        if not balanced:
            return torch.cat(parts, dim=1)
        c = x.shape[1] // 2
        chunks = [None] * (2 * W)
        for j, p in enumerate(parts):
            chunks[j], chunks[2 * W - 1 - j] = p[:, :c], p[:, c:]
        return torch.cat(chunks, dim=1)

    @staticmethod
    def backward(ctx, g):
        W, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        if ctx.balanced:
            c = g.shape[1] // (2 * W)
            per = [torch.cat((g[:, j * c : (j + 1) * c], g[:, (2 * W - 1 - j) * c : (2 * W - j) * c]), dim=1).contiguous()
                   for j in range(W)]
        else:
            c = g.shape[1] // W
            per = [g[:, j * c : (j + 1) * c].contiguous() for j in range(W)]
        out = torch.empty_like(per[r])
        dist.reduce_scatter(out, per, group=ctx.group)
        return out, None, None


class _RingPass(torch.autograd.Function):
    """K/V blocks passed around the ring; see module docstring (``alltoall`` method)."""

    @staticmethod
    def forward(ctx, q, k, v, group, scale, balanced):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        B, S, H, D = q.shape
        c = S // 2 if balanced else S
        my_chunks = (r, 2 * W - 1 - r) if balanced else (r,)
        out_parts = [None] * len(my_chunks)
        lse_parts = [None] * len(my_chunks)
        kv = torch.stack((k, v)).contiguous()
        nxt, prv = dist.get_global_rank(group, (r + 1) % W), dist.get_global_rank(group, (r - 1) % W)
        for step in range(W):
            j = (r - step) % W  # owner of the block we hold now
            kv_chunks = (j, 2 * W - 1 - j) if balanced else (j,)
            recv = None
            if step < W - 1:
                recv = torch.empty_like(kv)
                reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, kv, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)])
            for qi, a in enumerate(my_chunks):
                qa = q[:, qi * c : (qi + 1) * c]
                for ki, b in enumerate(kv_chunks):
                    if b > a:
                        continue
                    kb, vb = kv[0][:, ki * c : (ki + 1) * c], kv[1][:, ki * c : (ki + 1) * c]
                    o, l = ops.attention(qa, kb, vb, causal=(a == b), scale=scale, return_lse=True)
                    out_parts[qi], lse_parts[qi] = _merge(out_parts[qi], lse_parts[qi], o, l)
            if recv is not None:
                for w in reqs:
                    w.wait()
                kv = recv
        out = torch.cat([o.to(q.dtype) for o in out_parts], dim=1)
        lse = torch.cat(lse_parts, dim=2)  # [B,H,S]
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.group, ctx.scale, ctx.balanced = group, scale, balanced
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        group, scale, balanced = ctx.group, ctx.scale, ctx.balanced
        W, r = dist.get_world_size(group), dist.get_rank(group)
        S = q.shape[1]
        c = S // 2 if balanced else S
        my_chunks = (r, 2 * W - 1 - r) if balanced else (r,)
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)
        nxt, prv = dist.get_global_rank(group, (r + 1) % W), dist.get_global_rank(group, (r - 1) % W)
        do = do.contiguous()
        for step in range(W):
            j = (r - step) % W
            kv_chunks = (j, 2 * W - 1 - j) if balanced else (j,)
            for qi, a in enumerate(my_chunks):
                sl = slice(qi * c, (qi + 1) * c)
                for ki, b in enumerate(kv_chunks):
                    if b > a:
                        continue
                    ks = slice(ki * c, (ki + 1) * c)
                    gq, gk, gv = _attention_bwd_block(q[:, sl], kv[0][:, ks], kv[1][:, ks], out[:, sl], do[:, sl],
                                                      lse[:, :, sl], a == b, scale)
                    dq[:, sl] += gq.float()
                    dkv[0][:, ks] += gk.float()
                    dkv[1][:, ks] += gv.float()
            # pass the block and its gradient on (after the last step they are back at their owner + 1 ... so one extra hop)
            bundle = torch.cat((kv.float(), dkv)).contiguous()
            recv = torch.empty_like(bundle)
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, bundle, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]):
                w.wait()
            kv, dkv = recv[:2].to(k.dtype), recv[2:].contiguous()
        # after W hops every block (with its accumulated gradient) is home again
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def _attention_bwd_block(q, k, v, o, do, lse, causal, scale):
    """Gradients of one (query chunk, key chunk) block given the *final* output and log-sum-exp."""
    q, k, v, o, do = (t.contiguous() for t in (q, k, v, o, do))
    lse = lse.contiguous()
    if q.is_cuda:
        from torchtitan_b200.ops import cuda_ops

        if cuda_ops.attention_supported(q, k):
            return torch.ops.tt_b200.attention_bwd(q, k, v, o, do, lse, bool(causal), float(scale))
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2).repeat_interleave(g, 1), v.float().transpose(1, 2).repeat_interleave(g, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1 + (Sk - Sq))
        s = s.masked_fill(mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dof, of = do.float().transpose(1, 2), o.float().transpose(1, 2)
    delta = (dof * of).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(B, Hkv, g, Sk, D).sum(2)
    dv = dv.view(B, Hkv, g, Sk, D).sum(2)
    return dq.transpose(1, 2).to(q.dtype), dk.transpose(1, 2).to(k.dtype), dv.transpose(1, 2).to(v.dtype)


class RingAttention:
    def __init__(self, cp_mesh, rotate_method: str = "allgather", load_balancer: str | None = "headtail"):
        self.mesh, self.group = cp_mesh, cp_mesh.get_group()
        self.cp, self.rank = cp_mesh.size(), cp_mesh.get_local_rank()
        assert rotate_method in ("allgather", "alltoall")
        self.method, self.balanced = rotate_method, load_balancer is not None

    def _gather_ids(self, ids):
        """Per-token ids of the whole sequence in global order, from every rank's local shard ``[B, S_local]``."""
        W = self.cp
        parts = [torch.empty_like(ids) for _ in range(W)]
        dist.all_gather(parts, ids.contiguous(), group=self.group)
        if not self.balanced:
            return torch.cat(parts, dim=1)
        c = ids.shape[1] // 2
        chunks = [None] * (2 * W)
        for j, p in enumerate(parts):
            chunks[j], chunks[2 * W - 1 - j] = p[:, :c], p[:, c:]
        return torch.cat(chunks, dim=1)

    def __call__(self, q, k, v, *, scale=None, doc_ids=None, window=None, sinks=None):
        """``doc_ids`` are this rank's shard of the per-token document ids. Masks (documents, sliding window, sinks) need
        every query to see its whole key set in one softmax, which the ``allgather`` method gives; the ring method
        merges partial softmaxes and serves plain causal attention only."""
        masked = doc_ids is not None or window is not None or sinks is not None
        if masked and self.method == "alltoall":
            raise NotImplementedError("context parallel with document / window / sink masks needs "
                                      "parallelism.context_parallel_rotate_method='allgather'")
        scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if self.method == "alltoall":
            return _RingPass.apply(q, k, v, self.group, scale, self.balanced)
        K = _AllGatherKV.apply(k, self.group, self.balanced)
        V = _AllGatherKV.apply(v, self.group, self.balanced)
        docs = self._gather_ids(doc_ids) if doc_ids is not None else None
        W, r = self.cp, self.rank
        c = q.shape[1] if not self.balanced else q.shape[1] // 2
        owned = (r,) if not self.balanced else (r, 2 * W - 1 - r)
        outs = []
        for qi, a in enumerate(owned):
            end = (a + 1) * c
            # a sliding window never looks further back than window - 1 keys before the chunk's first query
            start = max(0, a * c - (window - 1)) if window is not None else 0
            kw = {}
            if masked:
                kw = dict(window=window, sinks=sinks, doc_ids=docs[:, start:end] if docs is not None else None)
            outs.append(ops.attention(q[:, qi * c : (qi + 1) * c], K[:, start:end], V[:, start:end], causal=True, scale=scale, **kw))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


def apply_cp_to_attention_module(attention_modules, cp_mesh, attn_backend: str = "sdpa", *, rotate_method: str = "allgather",
                                 load_balancer: str | None = "headtail") -> None:
    if attn_backend == "varlen":
        raise NotImplementedError("Varlen attention is not supported with CP.")
    ring = RingAttention(cp_mesh, rotate_method, load_balancer)
    for m in attention_modules:
        m.ring = ring
    logger.info(f"Applied Context Parallel (degree {cp_mesh.size()}, rotate={rotate_method}, balancer={load_balancer})")

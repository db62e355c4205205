"""Paged-KV generation engine for the framework's own decoder models.

It runs the *training* model object (``Decoder`` with ``GQAttention`` blocks: llama3, qwen3 dense and
MoE, llama4) for inference: a packed prefill of all prompts in one pass (document-masked flash
attention), then batched single-token decode steps over a block-table KV cache with the paged decode
kernel and the top-p sampler. Because projections, norms, RoPE and the log-softmax are the same
kernels the trainer uses, the generator's per-token log-probabilities match the trainer's recomputed
ones to rounding, which is the property the reference obtains by registering its model inside vLLM
(torchtitan/experiments/rl/unified/models/vllm_wrapper.py:40-408, models/attention.py:20-225).

Samples of one prompt share the prompt's full KV blocks (reference-counted); only the partial tail
block is copied per sample. With ``cudagraph=True`` a decode step of a given batch size is captured
once in a CUDA graph and replayed (inputs live in static buffers), removing per-step launch overhead.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from torchtitan_b200 import ops
from torchtitan_b200.models.common.attention import AttentionMasks
from torchtitan_b200.ops import serving


class BlockAllocator:
    """Host-side free list with reference counts (blocks shared by samples of one prompt)."""

    def __init__(self, num_blocks: int):
        self.free = list(range(num_blocks - 1, -1, -1))
        self.refs = [0] * num_blocks

    def alloc(self) -> int:
        if not self.free:
            raise RuntimeError("KV cache exhausted: raise gpu_memory_limit or lower the batch / max_tokens")
        b = self.free.pop()
        self.refs[b] = 1
        return b

    def share(self, b: int) -> int:
        self.refs[b] += 1
        return b

    def release(self, b: int) -> None:
        self.refs[b] -= 1
        if self.refs[b] == 0:
            self.free.append(b)

    @property
    def available(self) -> int:
        return len(self.free)


class PagedKVCache:
    def __init__(self, *, n_layers: int, num_blocks: int, block_size: int, n_kv_heads: int, head_dim: int, dtype, device):
        self.block_size, self.num_blocks = block_size, num_blocks
        shape = (num_blocks, block_size, n_kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.alloc = BlockAllocator(num_blocks)

    def copy_block(self, src: int, dst: int) -> None:
        for k, v in zip(self.k, self.v):
            k[dst].copy_(k[src])
            v[dst].copy_(v[src])

    @staticmethod
    def bytes_per_block(n_layers, block_size, n_kv_heads, head_dim, dtype) -> int:
        return 2 * n_layers * block_size * n_kv_heads * head_dim * torch.empty((), dtype=dtype).element_size()


@dataclass
class _Seq:
    prompt: int                 # index of the prompt this sample belongs to
    blocks: list[int]
    length: int                 # tokens whose KV is in the cache
    tokens: list[int]
    logprobs: list[float]
    done: bool = False
    hit_eos: bool = False


class GenerationEngine:
    def __init__(self, model, *, block_size: int = 16, num_blocks: int = 4096, max_batch: int = 512,
                 cudagraph: bool = False, eos_id: int | None = None):
        self.model = model
        p = next(model.parameters())
        self.device, self.dtype = p.device, p.dtype
        att = next(iter(model.layers.values())).attention
        self.n_kv_heads, self.head_dim = att.n_kv_heads, att.head_dim
        self.cache = PagedKVCache(n_layers=len(model.layers), num_blocks=num_blocks, block_size=block_size,
                                  n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, dtype=self.dtype, device=self.device)
        self.block_size, self.max_batch, self.eos_id = block_size, max_batch, eos_id
        self.cudagraph = cudagraph and self.device.type == "cuda"
        self._graphs: dict[tuple[int, int], tuple] = {}
        self.decode_steps = 0
        self.weight_half = 0   # which half of a double-buffered parameter arena the model currently reads

    # ---- one pass over the blocks with cache reads/writes -----------------------------------------
    def _attention(self, att, x, positions, layer: int, meta):
        T = x.shape[1]
        q = att.wq(x).view(1, T, -1, att.head_dim)
        k = att.wk(x).view(1, T, -1, att.head_dim)
        v = att.wv(x).view(1, T, -1, att.head_dim)
        if att.q_norm is not None:
            q, k = att.q_norm(q), att.k_norm(k)
        if att.use_rope:
            table = self.model.freqs_cis
            q = ops.rope(q, table, positions, att.rope_layout)
            k = ops.rope(k, table, positions, att.rope_layout)
        serving.kv_cache_write(self.cache.k[layer], self.cache.v[layer], k[0], v[0], meta["slots"])
        scale = att.scaling if att.scaling is not None else att.head_dim**-0.5
        if meta["prefill"]:
            out = ops.attention(q, k, v, causal=True, scale=scale, doc_ids=meta["doc_ids"])
        else:
            out = serving.paged_attention_decode(q[0], self.cache.k[layer], self.cache.v[layer], meta["block_tables"],
                                                 meta["context_lens"], scale).unsqueeze(0)
        return att.wo(out.reshape(1, T, -1))

    def _forward(self, tokens, positions, meta, last_index=None):
        m = self.model
        h = m.tok_embeddings(tokens)
        for li, layer in enumerate(m.layers.values()):
            h = h + self._attention(layer.attention, layer.attention_norm(h), positions, li, meta)
            ff = layer.moe if getattr(layer, "moe_enabled", False) else layer.feed_forward
            h = h + ff(layer.ffn_norm(h))
        if last_index is not None:
            h = h[:, last_index]
        return m.output(m.norm(h))[0]

    # ---- public ------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: list[list[int]], *, n_samples: int, max_tokens: int, temperature: float, top_p: float,
                 generator: torch.Generator | None = None) -> list[_Seq]:
        """Returns ``len(prompts) * n_samples`` sequences, samples of one prompt adjacent."""
        dev, bs = self.device, self.block_size
        was_training = self.model.training
        self.model.eval()
        try:
            # -- prefill: all prompts packed in one row -------------------------------------------------
            toks, pos, doc, slots, last = [], [], [], [], []
            prompt_blocks = []
            for i, p in enumerate(prompts):
                nblk = (len(p) + bs - 1) // bs
                blks = [self.cache.alloc.alloc() for _ in range(nblk)]
                prompt_blocks.append(blks)
                toks += p
                pos += range(len(p))
                doc += [i] * len(p)
                slots += [blks[t // bs] * bs + t % bs for t in range(len(p))]
                last.append(len(toks) - 1)
            T = len(toks)
            pad = -T % 128 if dev.type == "cuda" else 0      # the flash kernel works on 128-token tiles
            scratch = None
            if pad:
                scratch = self.cache.alloc.alloc()            # padded tokens write into a throw-away block
                toks += [0] * pad
                pos += range(pad)
                doc += [len(prompts)] * pad
                slots += [scratch * bs + (t % bs) for t in range(pad)]
            t_ = lambda x, dt: torch.tensor(x, dtype=dt, device=dev)  # noqa: E731
            meta = {"prefill": True, "slots": t_(slots, torch.int32), "doc_ids": t_(doc, torch.int32).unsqueeze(0)}
            logits = self._forward(t_(toks, torch.long).unsqueeze(0), t_(pos, torch.int32).unsqueeze(0), meta,
                                   last_index=t_(last, torch.long))
            if scratch is not None:
                self.cache.alloc.release(scratch)

            # -- fork samples: share full prompt blocks, copy the partial tail ----------------------------
            seqs: list[_Seq] = []
            for i, p in enumerate(prompts):
                full = len(p) // bs
                for s in range(n_samples):
                    blks = [self.cache.alloc.share(b) for b in prompt_blocks[i][:full]]
                    if len(p) % bs:
                        nb = self.cache.alloc.alloc()
                        self.cache.copy_block(prompt_blocks[i][full], nb)
                        blks.append(nb)
                    seqs.append(_Seq(prompt=i, blocks=blks, length=len(p), tokens=[], logprobs=[]))
                for b in prompt_blocks[i]:
                    self.cache.alloc.release(b)
            first_logits = logits.repeat_interleave(n_samples, dim=0)

            # -- decode -------------------------------------------------------------------------------------
            active = list(range(len(seqs)))
            cur_logits = first_logits
            for step in range(max_tokens):
                u = torch.rand(len(active), device=dev, generator=generator) if generator is not None or dev.type != "cuda" \
                    else torch.rand(len(active), device=dev)
                tok, lp = serving.sample_top_p(cur_logits, temperature, top_p, u)
                tok_l, lp_l = tok.tolist(), lp.tolist()
                nxt = []
                for j, si in enumerate(active):
                    s = seqs[si]
                    s.tokens.append(tok_l[j])
                    s.logprobs.append(lp_l[j])
                    if self.eos_id is not None and tok_l[j] == self.eos_id:
                        s.done = s.hit_eos = True
                    elif len(s.tokens) >= max_tokens:
                        s.done = True
                    else:
                        nxt.append((si, tok_l[j]))
                if not nxt:
                    break
                active = [si for si, _ in nxt]
                cur_logits = self._decode_step(seqs, active, [t for _, t in nxt])
            return seqs
        finally:
            for s in locals().get("seqs", []):
                for b in s.blocks:
                    self.cache.alloc.release(b)
                s.blocks = []
            if was_training:
                self.model.train()

    def _decode_step(self, seqs, active, last_tokens):
        dev, bs = self.device, self.block_size
        B = len(active)
        slots, ctx = [], []
        for si in active:
            s = seqs[si]
            if s.length % bs == 0 and s.length // bs >= len(s.blocks):
                s.blocks.append(self.cache.alloc.alloc())
            slots.append(s.blocks[s.length // bs] * bs + s.length % bs)
            s.length += 1
            ctx.append(s.length)
        maxb = max(len(seqs[si].blocks) for si in active)
        maxb = -(-maxb // 8) * 8                        # few distinct table widths => few captured graphs
        bt = [seqs[si].blocks + [0] * (maxb - len(seqs[si].blocks)) for si in active]
        t_ = lambda x, dt: torch.tensor(x, dtype=dt, device=dev)  # noqa: E731
        tokens, positions = t_(last_tokens, torch.long).unsqueeze(0), t_([c - 1 for c in ctx], torch.int32).unsqueeze(0)
        meta = {"prefill": False, "slots": t_(slots, torch.int32), "block_tables": t_(bt, torch.int32),
                "context_lens": t_(ctx, torch.int32)}
        self.decode_steps += 1
        if not self.cudagraph:
            return self._forward(tokens, positions, meta)
        key = (B, maxb, self.weight_half)     # captured graphs hold parameter addresses: one set per arena half
        if key not in self._graphs:
            static = {"tokens": tokens.clone(), "positions": positions.clone(),
                      "meta": {k: (v.clone() if torch.is_tensor(v) else v) for k, v in meta.items()}}
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):                      # warm-up outside capture
                    self._forward(static["tokens"], static["positions"], static["meta"])
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self._forward(static["tokens"], static["positions"], static["meta"])
            self._graphs[key] = (g, static, out)
        g, static, out = self._graphs[key]
        static["tokens"].copy_(tokens)
        static["positions"].copy_(positions)
        for k, v in meta.items():
            if torch.is_tensor(v):
                static["meta"][k].copy_(v)
        g.replay()
        return out

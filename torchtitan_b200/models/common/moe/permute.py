"""Index generation for regrouping all-to-all output by local expert.

After expert-parallel dispatch a rank holds rows ordered ``[source rank][local expert]``;
grouped GEMMs want ``[local expert][source rank]`` with every expert's block padded to a
multiple of ``alignment`` rows. ``generate_permute_indices`` returns, for each padded output
row, the input row it copies from (or -1 for padding).

Parity: torchtitan/models/common/moe/kernels.py:108-218 (CPU definition ``fill_indices_cpu``
and the wrapper's contract: int32 counts ``[ranks * experts_per_rank]``, output of length
``max_len`` filled with -1, ``m_sizes``/``m_offsets`` per local expert). ``fill_indices`` is the
same table computed with tensor operations only (prefix sums and one scatter), so that on a GPU nothing
is read on the host; the reference's is a Triton kernel (kernels.py:17-105).
"""

from __future__ import annotations

import torch


def fill_indices_cpu(tokens_per_expert_group, start_index_values, write_offsets,
                     experts_per_rank: int, num_ranks: int, max_len: int):
    out = torch.full((max_len,), -1, dtype=torch.int32)
    for e in range(experts_per_rank):
        w = int(write_offsets[e])
        for r in range(num_ranks):
            i = r * experts_per_rank + e
            n = int(tokens_per_expert_group[i])
            s = int(start_index_values[i])
            if n > 0 and w < max_len:
                end = min(w + n, max_len)
                out[w:end] = torch.arange(s, s + (end - w), dtype=torch.int32)
            w += n
    return out


def fill_indices(tokens_per_expert_group, start_index_values, write_offsets,
                 experts_per_rank: int, num_ranks: int, max_len: int):
    """Same result as :func:`fill_indices_cpu` on the tensors' own device, without loops or host reads. Output row ``p``
    lies in the block of expert ``e`` (last write offset <= p) at offset ``q``; the source rank is the first whose running
    total of rows for ``e`` exceeds ``q``; past the last rank the row is padding."""
    t = tokens_per_expert_group.to(torch.int64)
    dev = t.device
    by_rank = t.view(num_ranks, experts_per_rank)
    upto = torch.cumsum(by_rank, 0)                                    # [R, E] rows of expert e from ranks <= r
    p = torch.arange(max_len, device=dev)
    wo = write_offsets.to(torch.int64)
    e = (torch.searchsorted(wo, p, right=True) - 1).clamp_min(0)
    q = p - wo[e]
    r = (upto.t()[e] <= q.unsqueeze(1)).sum(1)                         # [max_len]; == R: padding
    valid = r < num_ranks
    r = r.clamp_max(num_ranks - 1)
    chunk = r * experts_per_rank + e
    src = start_index_values.to(torch.int64)[chunk] + q - (upto - by_rank).reshape(-1)[chunk]
    return torch.where(valid, src, torch.full_like(src, -1)).to(torch.int32)


def fill_indices_wrapper(tokens_per_expert_group, start_index_values, write_offsets, experts_per_rank: int,
                         num_ranks: int, max_len: int, block_size: int = 128, max_blocks: int = 1024):
    """The reference's name for the device version (its launch parameters are accepted and unused)."""
    return fill_indices(tokens_per_expert_group, start_index_values, write_offsets, experts_per_rank, num_ranks, max_len)


def generate_permute_indices(tokens_per_expert_group, experts_per_rank: int, num_ranks: int,
                             max_len: int, alignment: int, use_cpu: bool | None = None):
    """Returns (permuted_indices [max_len] int32, m_sizes [experts_per_rank] int32,
    m_offsets [experts_per_rank] int32 = inclusive cumsum of m_sizes)."""
    t = tokens_per_expert_group
    start_index_values = torch.cumsum(t, 0) - t
    total_per_expert = t.view(num_ranks, experts_per_rank).sum(0)
    total_per_expert = torch.clamp_min(total_per_expert, alignment)
    m_sizes = ((total_per_expert + alignment - 1) // alignment * alignment).to(torch.int32)
    m_offsets = torch.cumsum(m_sizes, 0)
    write_offsets = m_offsets - m_sizes
    if use_cpu:
        idx = fill_indices_cpu(t.cpu(), start_index_values.cpu(), write_offsets.cpu(), experts_per_rank, num_ranks, max_len).to(t.device)
    else:
        idx = fill_indices(t, start_index_values, write_offsets, experts_per_rank, num_ranks, max_len)
    return idx, m_sizes, m_offsets.to(torch.int32)

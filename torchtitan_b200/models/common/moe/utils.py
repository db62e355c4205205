"""Row-alignment helpers of the expert layers under the reference's module name
(torchtitan/models/common/moe/utils.py:21-123).

The grouped GEMMs want every expert's block of rows to start at a multiple of some alignment. The dispatchers of this
framework take it from :func:`moe.group_alignment` (64 for the bf16 kernel, 128 for block-scaled MXFP8, 8 on the CPU);
``set_token_group_alignment_size_m`` raises that floor, which is what quantisation converters written against the
reference call. ``indices_padding_wrapper`` pads the token groups of a per-expert function with the permutation table of
``permute.py``, without reading the group sizes on the host."""

from __future__ import annotations

from typing import Callable, Literal

import torch

from .permute import generate_permute_indices

ValidTokenGroupAlignmentSize = Literal[8, 16, 32, 64, 128]
MXFP8_GROUP_ALIGNMENT_SIZE = 32
TOKEN_GROUP_ALIGN_SIZE_M: int = 8


def set_token_group_alignment_size_m(alignment_size: int) -> None:
    """Smallest alignment the dispatchers may use from now on: 8 for bf16, 16 for float8, 32 for MXFP8 in the
    reference's terms; the native kernels ask for more by themselves."""
    global TOKEN_GROUP_ALIGN_SIZE_M
    if alignment_size not in (8, 16, 32, 64, 128):
        raise ValueError(f"token group alignment must be one of 8, 16, 32, 64, 128; got {alignment_size}")
    TOKEN_GROUP_ALIGN_SIZE_M = int(alignment_size)


def get_mxfp8_pad_multiple() -> int | None:
    return MXFP8_GROUP_ALIGNMENT_SIZE if TOKEN_GROUP_ALIGN_SIZE_M == MXFP8_GROUP_ALIGNMENT_SIZE else None


def maybe_align_num_tokens_for_mxfp8(num_tokens: int) -> int:
    m = get_mxfp8_pad_multiple()
    return num_tokens if m is None else -(-num_tokens // m) * m


def _permute(x: torch.Tensor, num_tokens_per_expert: torch.Tensor, ep_degree: int, num_local_experts: int):
    """Rows ordered ``[source rank][local expert]`` -> ``[local expert][source rank]`` with every expert's block padded to
    the alignment; returns (shape with the extra zero row, padded rows, table, padded counts)."""
    align = TOKEN_GROUP_ALIGN_SIZE_M
    max_len = -(-(x.shape[0] + num_local_experts * align) // align) * align
    with torch.no_grad():
        table, padded_counts, _ = generate_permute_indices(num_tokens_per_expert, num_local_experts, ep_degree, max_len, align)
    x = torch.vstack((x, x.new_zeros((1, x.shape[-1]))))           # index -1 of the table reads this zero row
    return x.shape, x[table.long(), :], table, padded_counts


def _unpermute(out: torch.Tensor, input_shape, permuted_indices: torch.Tensor) -> torch.Tensor:
    back = out.new_zeros(input_shape)
    back[permuted_indices.long(), :] = out
    return back[:-1]


def indices_padding_wrapper(func: Callable) -> Callable:
    """``func(w1, w2, w3, x, counts)`` sees padded groups; its output comes back in the original row order."""

    def wrapper(w1, w2, w3, x, num_tokens_per_expert):
        n_local = w1.shape[0]
        shape, xp, table, counts = _permute(x, num_tokens_per_expert, num_tokens_per_expert.shape[0] // n_local, n_local)
        return _unpermute(func(w1, w2, w3, xp, counts), shape, table)

    return wrapper

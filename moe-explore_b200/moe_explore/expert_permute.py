"""Routing metadata and the stand-alone permute helpers.

Same names and return types as the reference (src/moe_explore/expert_permute.py:8-68).  The
sort is the library's stable counting sort, so ``indices`` equals
``torch.sort(flat_expert_indices, stable=True).indices`` bit for bit (the reference calls a
non-stable ``argsort``, whose order inside an expert is unspecified).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple, Union

import torch

from moe_explore import _native
from moe_explore.functional.scale_and_reduce import scale_and_reduce
from moe_explore.routing_plan import build_routing_plan


@dataclass
class GroupedTokens:
    tokens: torch.Tensor
    group_indices: torch.Tensor
    indices: torch.Tensor


@dataclass
class PermToGroupIndices:
    group_indices: torch.Tensor
    indices: torch.Tensor


def get_token_indices(expert_indices: torch.Tensor, topk: int, num_experts: int, zero_prefix: bool = False) -> PermToGroupIndices:
    """``expert_indices`` int64 [T, topk] -> per-expert row ranges and the permutation that sorts
    the flat (token, slot) positions by expert (expert_permute.py:19-41).

    ``zero_prefix=True``: ``group_indices`` is int32 [E+1] starting at 0; otherwise the inclusive
    cumulative counts, int64 [E] (what ``counts.cumsum`` yields in the reference)."""
    plan = build_routing_plan(expert_indices, num_experts, topk, want_perm=True)
    if zero_prefix:
        groups = plan.group_indices
    else:
        groups = plan.group_indices[1:].to(torch.int64)
    return PermToGroupIndices(group_indices=groups, indices=plan.perm)


def row_gather(tokens: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``out[r] = tokens[indices[r]]`` (triton_kernels/row_gather_scatter.py:36-58)."""
    _native.require_cuda(tokens, indices)
    assert tokens.dim() == 2 and indices.dim() == 1
    out = torch.empty(indices.numel(), tokens.size(1), dtype=tokens.dtype, device=tokens.device)
    _native.unpad_rows(tokens.contiguous(), indices.to(torch.int32), out)
    return out


def row_scatter(tokens: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``out[indices[r]] = tokens[r]``; ``indices`` must be a permutation
    (triton_kernels/row_gather_scatter.py:91-116)."""
    _native.require_cuda(tokens, indices)
    assert tokens.dim() == 2 and indices.dim() == 1 and indices.numel() == tokens.size(0)
    inverse = torch.empty(indices.numel(), dtype=torch.int32, device=tokens.device)
    inverse[indices] = torch.arange(indices.numel(), dtype=torch.int32, device=tokens.device)
    out = torch.empty_like(tokens)
    _native.unpad_rows(tokens.contiguous(), inverse, out)
    return out


def expert_input_permute(tokens: torch.Tensor, expert_indices: torch.Tensor, num_experts: int, topk: int) -> GroupedTokens:
    """Gather token rows into expert order (expert_permute.py:43-56)."""
    found = get_token_indices(expert_indices, topk, num_experts, zero_prefix=True)
    grouped = row_gather(tokens, found.indices // topk)
    return GroupedTokens(tokens=grouped, group_indices=found.group_indices, indices=found.indices)


def expert_output_permute(grouped_tokens: GroupedTokens, expert_scores: torch.Tensor, topk: int,
                          output_shape: Union[Tuple[int], torch.Size]) -> torch.Tensor:
    """Scatter expert-ordered rows back to (token, slot) order and fold the slots with the router
    weights (expert_permute.py:58-68)."""
    tokens = row_scatter(grouped_tokens.tokens, grouped_tokens.indices)
    return scale_and_reduce(tokens, expert_scores, expert_scores.size(0), topk, tokens.size(1))

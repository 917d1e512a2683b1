"""Routing plan: everything the expert-compute kernels need to know about one routing decision.

Built by one call into the native routing-metadata kernels (histogram, prefix sums, stable
permutation, inverse, padded row layout, tile -> expert map).  No host synchronisation: buffer
sizes come from worst-case bounds, the number of tiles actually in use stays on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from moe_explore import _native


@dataclass
class RoutingPlan:
    num_rows: int                 # R = T * topk routed rows
    num_experts: int
    topk: int
    padded_rows: int              # RP: row count of every padded expert-sorted buffer
    group_indices: torch.Tensor   # int32 [E+1] exclusive prefix of per-expert counts
    perm: Optional[torch.Tensor]  # int64 [R]  stable argsort of the flat expert ids
    pad_offsets: torch.Tensor     # int32 [E+1] padded row offset of each expert
    row_src: torch.Tensor         # int32 [RP] flat position held by padded row p, -1 for padding
    dst_row: torch.Tensor         # int32 [R]  padded row of flat position j
    mtile_expert: torch.Tensor    # int32 [RP/128] expert of each 128-row tile
    tile_pairs: torch.Tensor      # int32 [RP/128 + E + 1] pair list (first tile | expert << 20 | two tiles << 31), then
                                  # from index RP/128 the exclusive prefix of the per-expert pair counts
    num_mtiles: torch.Tensor      # int32 [2]  {tiles in use, tile pairs in use}
    status: torch.Tensor          # int32 [1]  device status word shared by the kernels of this plan

    def check(self) -> None:
        """Synchronise and raise if any kernel that used this plan reported a problem."""
        _native.check_status(self.status)


def _alloc(num_rows: int, num_experts: int, device, want_perm: bool):
    rp = _native.padded_rows_bound(num_rows, num_experts)
    i32 = dict(dtype=torch.int32, device=device)
    return dict(
        padded_rows=rp,
        group_indices=torch.empty(num_experts + 1, **i32),
        perm=torch.empty(num_rows, dtype=torch.int64, device=device) if want_perm else None,
        pad_offsets=torch.empty(num_experts + 1, **i32),
        row_src=torch.empty(rp, **i32),
        dst_row=torch.empty(num_rows, **i32),
        mtile_expert=torch.empty(rp // _native.TILE_M, **i32),
        tile_pairs=torch.empty(rp // _native.TILE_M + num_experts + 1, **i32),
        num_mtiles=torch.empty(2, **i32),
        status=torch.zeros(1, **i32),
    )


def build_routing_plan(expert_indices: torch.Tensor, num_experts: int, topk: int, want_perm: bool = True) -> RoutingPlan:
    """``expert_indices``: int64 [T, topk] (or flat [T*topk]) expert id per (token, slot)."""
    _native.require_cuda(expert_indices)
    assert expert_indices.dtype is torch.int64, "expert indices must be int64 (what torch.topk returns)"
    flat = expert_indices.reshape(-1).contiguous()
    bufs = _alloc(flat.numel(), num_experts, flat.device, want_perm)
    ws = torch.empty(max(_native.routing_workspace_bytes(flat.numel(), num_experts), 16), dtype=torch.uint8,
                     device=flat.device)
    _native.routing_metadata(flat, num_experts, bufs["group_indices"], bufs["perm"], bufs["pad_offsets"],
                             bufs["row_src"], bufs["dst_row"], bufs["mtile_expert"], bufs["tile_pairs"],
                             bufs["num_mtiles"], bufs["status"], ws)
    return RoutingPlan(num_rows=flat.numel(), num_experts=num_experts, topk=topk, **bufs)


def plan_from_groups(group_indices: torch.Tensor, num_rows: int) -> RoutingPlan:
    """Plan for rows that are already grouped: ``group_indices`` int32 [E+1] exclusive prefix."""
    _native.require_cuda(group_indices)
    assert group_indices.dtype is torch.int32 and group_indices.dim() == 1
    num_experts = group_indices.numel() - 1
    bufs = _alloc(num_rows, num_experts, group_indices.device, want_perm=False)
    bufs["group_indices"] = group_indices.contiguous()
    _native.layout_from_groups(bufs["group_indices"], num_rows, num_experts, bufs["pad_offsets"], bufs["row_src"],
                               bufs["dst_row"], bufs["mtile_expert"], bufs["tile_pairs"], bufs["num_mtiles"])
    return RoutingPlan(num_rows=num_rows, num_experts=num_experts, topk=1, **bufs)

"""Routing plan: everything the expert-compute kernels need to know about one routing decision.

Built by one call into the native routing-metadata kernels (histogram, prefix sums, stable
permutation, inverse, padded row layout, tile -> expert map).  No host synchronisation: buffer
sizes come from worst-case bounds, the number of tiles actually in use stays on the device.

Status word.  Every kernel of this package that can detect a problem on the device (an expert id
out of range, metadata that does not fit the call, a bounded wait that ran out) records a code in
ONE int32 per device, ``device_status(device)``, shared by all plans built on that device; the
first code wins and the word stays set until it is read with ``check_device_status``.  Nothing
reads it on the hot path (that would be a host synchronisation per step): callers check it once
per step or per logging interval -- ``check_device_status()`` -- and must not trust the outputs
of a step after which it raised.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from moe_explore import _native

_DEVICE_STATUS: Dict[int, torch.Tensor] = {}


def device_status(device=None) -> torch.Tensor:
    """The int32 [1] status word of ``device`` (created zeroed on first use)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    word = _DEVICE_STATUS.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _DEVICE_STATUS[index] = word
    return word


def check_device_status(device=None, reset: bool = True) -> int:
    """Synchronise, read the device's status word (clearing it when ``reset``) and raise
    ``MoeNativeError`` if a kernel reported a problem since the last check.  A wave barrier that gave
    up (code 4: the launch completed correctly, only unsynchronised) is a warning, not an error.
    Returns the code."""
    return _report(_native.read_status(device_status(device), reset=reset))


def _report(code: int) -> int:
    if code == 0:
        return 0
    if code == _native.STATUS_WAVE_FALLBACK:
        warnings.warn("libmoe_sm100: the wave barrier of a grouped GEMM ran out (its persistent workers were not all "
                      "resident, e.g. another kernel held SMs); the launch finished unsynchronised, results are valid")
        return code
    if code == _native.STATUS_BAD_EXPERT_ID:
        raise _native.MoeNativeError("routing", -1, "an expert id outside [0, num_experts) reached the routing "
                                     "metadata; such (token, slot) pairs were dropped from the layer's output")
    if code == _native.STATUS_BAD_LAYOUT:
        raise _native.MoeNativeError("routing", -1, "routing metadata does not describe the rows it was used with")
    raise _native.MoeNativeError("kernel", -4, f"a device-side bounded wait ran out (code {code}); the outputs of "
                                 "that launch are incomplete")


@dataclass
class RoutingPlan:
    num_rows: int                 # R = T * topk routed rows
    num_experts: int
    topk: int
    padded_rows: int              # RP: row count of every padded expert-sorted buffer
    group_indices: torch.Tensor   # int32 [E+1] exclusive prefix of per-expert counts
    perm: Optional[torch.Tensor]  # int64 [R]  stable argsort of the flat expert ids (-1 past the rows kept)
    pad_offsets: torch.Tensor     # int32 [E+1] padded row offset of each expert
    row_src: torch.Tensor         # int32 [RP] flat position held by padded row p, -1 for padding
    dst_row: torch.Tensor         # int32 [R]  padded row of flat position j (-1: dropped, expert id out of range)
    mtile_expert: torch.Tensor    # int32 [RP/128] expert of each 128-row tile
    tile_pairs: torch.Tensor      # int32 [RP/128 + E + 1] pair list (first tile | expert << 20 | two tiles << 31), then
                                  # from index RP/128 the exclusive prefix of the per-expert pair counts
    num_mtiles: torch.Tensor      # int32 [4]  {tiles in use, tile pairs in use, RP/128, 0}
    status: torch.Tensor          # int32 [1]  the device's status word (shared, see the module docstring)

    def check(self) -> None:
        """Synchronise and raise if any kernel reported a problem through this plan's status word."""
        _report(_native.read_status(self.status, reset=True))


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
        num_mtiles=torch.empty(4, **i32),
        status=device_status(device),
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
    """Plan for rows that are already grouped: ``group_indices`` int32 [E+1] exclusive prefix of ``num_rows``.
    A prefix that does not run monotonically from 0 to ``num_rows`` is reported through the status word."""
    _native.require_cuda(group_indices)
    assert group_indices.dtype is torch.int32 and group_indices.dim() == 1
    num_experts = group_indices.numel() - 1
    bufs = _alloc(num_rows, num_experts, group_indices.device, want_perm=False)
    bufs["group_indices"] = group_indices.contiguous()
    _native.layout_from_groups(bufs["group_indices"], num_rows, num_experts, bufs["pad_offsets"], bufs["row_src"],
                               bufs["dst_row"], bufs["mtile_expert"], bufs["tile_pairs"], bufs["num_mtiles"],
                               bufs["status"])
    return RoutingPlan(num_rows=num_rows, num_experts=num_experts, topk=1, **bufs)

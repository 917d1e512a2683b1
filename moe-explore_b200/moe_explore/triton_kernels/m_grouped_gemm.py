"""Ragged M-grouped GEMM with optional fused row gather / scatter and activation epilogue.

Drop-in for the reference's Triton wrapper (src/moe_explore/triton_kernels/m_grouped_gemm.py:16-31,
332-393): same ``MGroupedGEMMParams`` fields and the same ``m_grouped_gemm(token, params,
autotune_mode=None)`` call.  The module keeps its reference path although nothing here is Triton:
the contraction runs on the library's tcgen05 kernel over the padded expert-sorted layout.
``autotune_mode`` is accepted and ignored (tile shapes are fixed at build time).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from moe_explore import _native
from moe_explore.functional.activation import is_glu
from moe_explore.routing_plan import plan_from_groups


@dataclass
class MGroupedGEMMParams:
    weight: torch.Tensor                      # [E, K, N]
    group_indices: torch.Tensor               # int32 [E+1], exclusive prefix of rows per expert
    permute_indices: Optional[torch.Tensor]   # int64 [T*topk], required with gather or scatter
    gather: bool                              # input row of sorted position r is token[permute_indices[r] // topk]
    scatter: bool                             # output row of sorted position r is written at permute_indices[r]
    # With gather or scatter ``num_tokens`` is the token count BEFORE routing (T); otherwise it is
    # simply the number of input rows.
    num_tokens: int
    topk: int
    shared_weight: Optional[torch.Tensor] = None
    scales: Optional[torch.Tensor] = None     # carried for the caller; not applied here
    activation: Optional[str] = None


def m_grouped_gemm(token: torch.Tensor, params: MGroupedGEMMParams, autotune_mode=None) -> torch.Tensor:
    """Rows [g[e], g[e+1]) of the (optionally gathered) input times ``weight[e]``, optional activation epilogue,
    optional scatter of the output rows.  As in the reference kernel the scatter happens inside the GEMM's epilogue
    (m_grouped_gemm.py:168-172): no un-scattered copy of the output exists.  The input rows are copied into
    128-row-aligned expert segments first (one HBM-bound pass) so that the GEMM loads whole tiles."""
    assert token.dim() == 2
    assert params.weight.dim() == 3
    assert token.size(1) == params.weight.size(1)
    if params.gather or params.scatter:
        assert params.permute_indices is not None
    _native.require_cuda(token, params.weight, params.group_indices)

    num_experts, k_dim, n_dim = params.weight.shape
    rows = params.num_tokens * params.topk if (params.gather or params.scatter) else params.num_tokens
    act = None if params.activation is None else str(params.activation)
    assert act in _native.ACT_CODES, f"Invalid activation: {act}"
    out_cols = n_dim // 2 if is_glu(act) else n_dim
    out = torch.empty(rows, out_cols, dtype=token.dtype, device=token.device)
    if rows == 0:
        return out

    plan = plan_from_groups(params.group_indices.to(torch.int32), rows)
    token = token.contiguous()
    weight = params.weight.contiguous()
    # padded row p holds sorted position r = row_src[p]; with gather or scatter its flat (token, slot) position is
    # perm[r]: the input row is token[perm[r] // topk], the output row perm[r]
    flat_of_row = None
    if params.gather or params.scatter:
        perm32 = params.permute_indices.to(torch.int32)
        flat_of_row = torch.where(plan.row_src >= 0, perm32[plan.row_src.clamp_min(0).long()], plan.row_src)
    in_rows = flat_of_row if params.gather else plan.row_src     # input row of padded row p (before // div)
    in_div = params.topk if params.gather else 1
    out_rows = flat_of_row if params.scatter else plan.row_src   # output row of padded row p
    # input rows into the padded layout with one copy kernel (the gather could ride on the GEMM's operand loads --
    # mgrouped_gemm_gather -- but four-row gather copies are several times slower than 128-row tile copies)
    a = torch.empty(plan.padded_rows, k_dim, dtype=token.dtype, device=token.device)
    _native.gather_rows(token, in_rows, plan.num_mtiles, a, in_div)
    if not is_glu(act):
        # element-wise epilogue: the rows are scattered to their final place by the stores of the GEMM itself
        _native.mgrouped_gemm_scatter(a, weight, out, out_rows, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles,
                                      plan.padded_rows, False, act, status=plan.status)
        return out
    # gated epilogue (two input columns per output column): output in the padded layout, then one un-pad pass
    y = torch.empty(plan.padded_rows, out_cols, dtype=token.dtype, device=token.device)
    _native.mgrouped_gemm(a, weight, y, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, False, act, plan.status)
    if params.scatter:
        src_of_out = torch.empty(rows, dtype=torch.int32, device=token.device)
        src_of_out[params.permute_indices] = plan.dst_row   # out[perm[r]] = y[dst_row[r]]
        _native.unpad_rows(y, src_of_out, out)
    else:
        _native.unpad_rows(y, plan.dst_row, out)
    return out

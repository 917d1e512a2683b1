"""The top-k mixture-of-experts layer.

``topk_moe_forward`` keeps the reference signature (src/moe_explore/functional/topk_moe.py:10-64)
and is differentiable with respect to the input, the router weight and both expert weight
tensors.  ``topk_moe_torch`` restates the reference's per-expert torch loop
(functional/topk_moe.py:67-102) with out-of-place ops so that autograd works; it is a
torch-on-the-same-device cross-check, not a fallback of ``topk_moe_forward``.
"""
from __future__ import annotations

import torch

from moe_explore.expert_compute import expert_compute
from moe_explore.functional.activation import activation
from moe_explore.params import MLPParams, MOEParams, TopkRouterParams
from moe_explore.router import fused_topk_router, router
from moe_explore.routing_plan import build_routing_plan


def _shared_expert(input: torch.Tensor, shared) -> torch.Tensor:
    """The shared-expert branch (functional/topk_moe.py:56-62): ``h = act(input @ up_weight) @ down_weight`` followed
    by ``h.sum(0)``.  With 3-D weights -- ``up_weight`` [S, d, I or 2I], ``down_weight`` [S, I, d], S shared experts
    -- ``sum(0)`` adds the S experts' outputs per token; that case runs on the grouped-GEMM kernels as a top-S layer
    in which every token is routed to every shared expert with weight one (differentiable like the routed experts).
    With 2-D weights the reference's ``sum(0)`` runs over the TOKENS and the resulting [d] vector is broadcast onto
    every row; that literal behaviour is kept, in torch ops."""
    up, down = shared.up_weight, shared.down_weight
    if up.dim() == 3:
        num_shared = up.size(0)
        T = input.size(0)
        indices = torch.arange(num_shared, device=input.device, dtype=torch.int64).repeat(T, 1)
        ones = torch.ones(T, num_shared, dtype=input.dtype, device=input.device)
        plan = build_routing_plan(indices, num_shared, num_shared, want_perm=False)
        return expert_compute(input, ones, up, down, plan, shared.activation)
    h = input @ up
    h = activation(h, shared.activation)
    h = h @ down
    return h.sum(0)


def topk_moe_forward(input: torch.Tensor, params: MOEParams, autotune_mode=None, *, fused_router: bool = False,
                     gather_in_gemm=None, fused_combine: bool = False) -> torch.Tensor:
    """The layer (functional/topk_moe.py:10-64).  ``autotune_mode`` is accepted and ignored.  Keyword-only additions:
    ``fused_router`` runs the router tail in one kernel with its own declared tie rule (see
    ``moe_explore.router.fused_topk_router``); ``gather_in_gemm`` / ``fused_combine`` as in ``expert_compute``."""
    ep: MLPParams = params.expert_params
    if fused_router and isinstance(params.router_params, TopkRouterParams):
        scores, indices = fused_topk_router(input, params.router_params)
    else:
        scores, indices = router(input, params.router_params)
    plan = build_routing_plan(indices, params.num_experts, params.topk, want_perm=False)
    out = expert_compute(input, scores, ep.weight1, ep.weight2, plan, ep.activation, gather_in_gemm=gather_in_gemm,
                         fused_combine=fused_combine)
    shared = getattr(params, "shared_expert_params", None)
    if shared is not None:
        out = out + _shared_expert(input, shared)
    return out


def topk_moe_torch(input: torch.Tensor, params: MOEParams, autotune_mode=None) -> torch.Tensor:
    ep: MLPParams = params.expert_params
    scores, indices = router(input, params.router_params)
    flat_scores = scores.reshape(-1, 1)
    flat_experts = indices.reshape(-1)
    order = torch.sort(flat_experts, stable=True).indices
    counts = torch.bincount(flat_experts, minlength=params.num_experts)
    ends = counts.cumsum(0).tolist()
    out = torch.zeros_like(input)
    start = 0
    for expert_id, end in enumerate(ends):
        if end == start:
            continue
        rows = order[start:end]
        tok = rows // params.topk
        h = activation(input[tok] @ ep.weight1[expert_id], ep.activation)
        y = (h @ ep.weight2[expert_id]) * flat_scores[rows]
        out = out.index_add(0, tok, y)
        start = end
    return out

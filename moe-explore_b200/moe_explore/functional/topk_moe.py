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
from moe_explore.params import MLPParams, MOEParams
from moe_explore.router import router
from moe_explore.routing_plan import build_routing_plan


def _shared_expert(input: torch.Tensor, shared) -> torch.Tensor:
    # Literal restatement of functional/topk_moe.py:57-62 (dense up -> activation -> down, summed
    # over rows and broadcast-added), kept as plain library matmuls.
    h = input @ shared.up_weight
    h = activation(h, shared.activation)
    h = h @ shared.down_weight
    return h.sum(0)


def topk_moe_forward(input: torch.Tensor, params: MOEParams, autotune_mode=None) -> torch.Tensor:
    ep: MLPParams = params.expert_params
    scores, indices = router(input, params.router_params)
    plan = build_routing_plan(indices, params.num_experts, params.topk, want_perm=False)
    out = expert_compute(input, scores, ep.weight1, ep.weight2, plan, ep.activation)
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

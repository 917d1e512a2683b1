"""Token -> expert routing.

Kept as plain torch ops on purpose: the reference computes its routing with the same ops
(src/moe_explore/router.py:9-54), so running them on the same device gives bit-identical
top-k indices and scores, which the expert-compute kernels downstream depend on.
``torch.compile`` decoration is dropped (no tracing compiler on this path).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from moe_explore.params import ErnieRouterParams, RouterParams, TopkRouterParams


def softmax(x: torch.Tensor) -> torch.Tensor:
    """fp32 softmax over the last dim (router.py:5-7)."""
    return F.softmax(x, dim=-1, dtype=torch.float32)


def router(input: torch.Tensor, params: RouterParams):
    """Dispatch on the parameter type (router.py:9-15). Returns (scores [T,k], indices [T,k] int64)."""
    if isinstance(params, TopkRouterParams):
        return topk_router(input, params)
    if isinstance(params, ErnieRouterParams):
        return ernie_router(input, params)
    raise ValueError(f"Unsupported router type: {type(params)}")


def topk_router(input: torch.Tensor, router_params: TopkRouterParams):
    """Linear logits -> (softmax ->) top-k (-> softmax over the k) (-> renormalise) (router.py:17-35)."""
    logits = input @ router_params.router_weight
    if router_params.softmax_before_topk:
        logits = softmax(logits)
    scores, indices = torch.topk(logits, k=router_params.topk, dim=-1, sorted=False)
    if not router_params.softmax_before_topk:
        scores = softmax(scores)
    if router_params.normalize_routing:
        scores = scores / scores.sum(dim=-1, keepdim=True)
    return scores.to(input.dtype), indices


def ernie_router(input: torch.Tensor, router_params: ErnieRouterParams):
    """All-fp32 router with a selection-only bias and clamp-normalised weights (router.py:37-54)."""
    assert router_params.router_weight.dtype is torch.float32
    with torch.autocast(device_type=input.device.type, enabled=False):
        probs = softmax(input.float() @ router_params.router_weight)
        _, indices = torch.topk(probs + router_params.bias, k=router_params.topk, dim=-1, sorted=False)
        picked = torch.gather(probs, dim=-1, index=indices)
        picked = picked / torch.clamp(picked.sum(dim=-1, keepdim=True), min=1e-12)
        return picked.to(input.dtype), indices

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


class _FusedTopk(torch.autograd.Function):
    """scores, indices = fused router tail of ``logits``; differentiable with respect to the logits."""

    @staticmethod
    def forward(ctx, logits, topk, softmax_before_topk, normalize_routing):
        from moe_explore import _native

        scores, indices, _ = _native.router_topk(logits, topk, softmax_before_topk, normalize_routing)
        ctx.save_for_backward(logits, indices)
        ctx.cfg = (softmax_before_topk, normalize_routing)
        ctx.mark_non_differentiable(indices)
        return scores, indices

    @staticmethod
    def backward(ctx, d_scores, _d_indices):
        # the scores as a differentiable torch function of the logits GIVEN the selection (gather, not top-k)
        logits, indices = ctx.saved_tensors
        softmax_before_topk, normalize_routing = ctx.cfg
        with torch.enable_grad():
            leaf = logits.detach().requires_grad_(True)
            if softmax_before_topk:
                picked = torch.gather(softmax(leaf), -1, indices)
            else:
                picked = softmax(torch.gather(leaf, -1, indices))
            if normalize_routing:
                picked = picked / picked.sum(dim=-1, keepdim=True)
            picked.to(logits.dtype).backward(d_scores)
        return leaf.grad, None, None, None


def fused_topk_router(input: torch.Tensor, router_params: TopkRouterParams):
    """``topk_router`` with everything after the logits GEMM in ONE kernel (softmax, top-k, softmax over the k,
    renormalisation, cast).  Opt-in: its tie rule is its own (equal logits are taken in ascending expert index; the
    k results come in descending score order, where ``torch.topk(sorted=False)`` leaves the order unspecified), so
    on inputs with tied logits among the selected values the indices can differ from ``topk_router``'s; without
    such ties the set of experts per token is the same and the scores agree to one rounding of the 16-bit type.
    (router.py:17-35)"""
    logits = input @ router_params.router_weight
    return _FusedTopk.apply(logits, router_params.topk, bool(router_params.softmax_before_topk),
                            bool(router_params.normalize_routing))


def ernie_router(input: torch.Tensor, router_params: ErnieRouterParams):
    """All-fp32 router with a selection-only bias and clamp-normalised weights (router.py:37-54)."""
    assert router_params.router_weight.dtype is torch.float32
    with torch.autocast(device_type=input.device.type, enabled=False):
        probs = softmax(input.float() @ router_params.router_weight)
        _, indices = torch.topk(probs + router_params.bias, k=router_params.topk, dim=-1, sorted=False)
        picked = torch.gather(probs, dim=-1, index=indices)
        picked = picked / torch.clamp(picked.sum(dim=-1, keepdim=True), min=1e-12)
        return picked.to(input.dtype), indices

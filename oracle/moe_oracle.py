"""CPU oracle for the top-k MoE expert-compute path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A plain-torch (fp32 by default, any device) restatement of the reference algorithm, function
by function.  Only the tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product package never does.

Parity status
  * forward path (router, routing metadata, activation, expert loop, scale-and-reduce):
    PINNED against outputs of the reference itself, generated in a container that holds the
    reference sources by tests/golden/make_golden.py and committed under tests/golden/.
  * permutation order inside one expert: the reference calls a non-stable ``argsort``
    (expert_permute.py:27); the canonical order here is the stable one.  The golden files pin
    that each expert's segment holds the same set of flat positions as the reference's.
  * backward: PARITY UNPINNED -- the reference has no backward pass (its torch loop raises under
    autograd because of an in-place scatter_reduce_).  Gradients are defined as torch.autograd
    of ``topk_moe`` below, cross-checked by finite differences in float64.

Reference citations are file:line inside arthurfeeney/moe-explore.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# router -- src/moe_explore/router.py
# --------------------------------------------------------------------------------------
def softmax_fp32(x: torch.Tensor) -> torch.Tensor:
    """router.py:5-7 -- softmax over the last dim computed in fp32."""
    return F.softmax(x, dim=-1, dtype=torch.float32)


def topk_router(x: torch.Tensor, router_weight: torch.Tensor, topk: int, softmax_before_topk: bool = True,
                normalize_routing: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """router.py:17-35 -- logits = x @ Wr; softmax before or after the top-k; optional renormalise;
    scores cast to x.dtype; indices int64 in torch.topk(sorted=False) order."""
    logits = x @ router_weight
    if softmax_before_topk:
        logits = softmax_fp32(logits)
    scores, indices = torch.topk(logits, k=topk, dim=-1, sorted=False)
    if not softmax_before_topk:
        scores = softmax_fp32(scores)
    if normalize_routing:
        scores = scores / scores.sum(dim=-1, keepdim=True)
    return scores.to(x.dtype), indices


def ernie_router(x: torch.Tensor, router_weight: torch.Tensor, bias: torch.Tensor, topk: int):
    """router.py:37-54 -- fp32 probabilities; bias used for selection only; clamp-normalised."""
    probs = softmax_fp32(x.float() @ router_weight)
    _, indices = torch.topk(probs + bias, k=topk, dim=-1, sorted=False)
    w = torch.gather(probs, dim=-1, index=indices)
    w = w / torch.clamp(w.sum(dim=-1, keepdim=True), min=1e-12)
    return w.to(x.dtype), indices


# --------------------------------------------------------------------------------------
# routing metadata -- src/moe_explore/expert_permute.py
# --------------------------------------------------------------------------------------
@dataclass
class TokenIndices:
    group_indices: torch.Tensor  # zero_prefix: int32 [E+1]; else inclusive cumsum int64 [E]
    indices: torch.Tensor        # int64 [T*k], stable order


def get_token_indices(expert_indices: torch.Tensor, topk: int, num_experts: int, zero_prefix: bool = False) -> TokenIndices:
    """expert_permute.py:19-41 -- argsort of the flattened ids (stable here), per-expert counts
    (histc there, bincount here: identical for integer ids in range), prefix sum."""
    flat = expert_indices.reshape(-1)
    indices = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    if zero_prefix:
        group = torch.zeros(num_experts + 1, dtype=torch.int32, device=flat.device)
        group[1:] = counts.cumsum(0)
    else:
        group = counts.cumsum(0)  # int32 cumsum promotes to int64, as in the reference
    return TokenIndices(group, indices)


def padded_layout(expert_indices: torch.Tensor, num_experts: int, tile: int = 128):
    """The padded expert-sorted row layout the CUDA kernels use (no reference counterpart):
    returns pad_offsets int32 [E+1], row_src int32 [pad_offsets[-1]] (-1 = padding),
    dst_row int32 [R], mtile_expert int32 [pad_offsets[-1] / tile]."""
    flat = expert_indices.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + tile - 1) // tile * tile
    pad_offsets = torch.zeros(num_experts + 1, dtype=torch.int64)
    pad_offsets[1:] = padded.cumsum(0)
    starts = torch.zeros(num_experts + 1, dtype=torch.int64)
    starts[1:] = counts.cumsum(0)
    row_src = torch.full((int(pad_offsets[-1]),), -1, dtype=torch.int32)
    dst_row = torch.empty(flat.numel(), dtype=torch.int32)
    for e in range(num_experts):
        c = int(counts[e])
        seg = order[int(starts[e]): int(starts[e]) + c]
        rows = torch.arange(int(pad_offsets[e]), int(pad_offsets[e]) + c, dtype=torch.int64)
        row_src[rows] = seg.to(torch.int32)
        dst_row[seg] = rows.to(torch.int32)
    mtile_expert = torch.repeat_interleave(torch.arange(num_experts, dtype=torch.int32), padded // tile)
    return pad_offsets.to(torch.int32), row_src, dst_row, mtile_expert


# --------------------------------------------------------------------------------------
# activation / scale-and-reduce -- src/moe_explore/functional/
# --------------------------------------------------------------------------------------
def activation(x: torch.Tensor, name: Optional[str]) -> torch.Tensor:
    """functional/activation.py:11-26 -- silu, exact gelu, or the gated forms on interleaved
    columns (gate = even columns, linear branch = odd columns)."""
    if name is None:
        return x
    if name == "silu":
        return F.silu(x)
    if name == "gelu":
        return F.gelu(x)
    assert name in ("swiglu", "geglu"), name
    gate, up = x[..., 0::2], x[..., 1::2]
    return (F.silu(gate) if name == "swiglu" else F.gelu(gate)) * up


def scale_and_reduce(y: torch.Tensor, scales: torch.Tensor, num_tokens: int, topk: int) -> torch.Tensor:
    """functional/scale_and_reduce.py:3-5."""
    return (y.view(num_tokens, topk, -1) * scales[..., None]).sum(1)


# --------------------------------------------------------------------------------------
# grouped matmul -- src/moe_explore/testing.py:9-50 (the reference's own test oracle)
# --------------------------------------------------------------------------------------
def grouped_matmul(a: torch.Tensor, weight: torch.Tensor, group_indices: torch.Tensor, permute_indices=None,
                   gather: bool = False, scatter: bool = False, topk: int = 1, act: Optional[str] = None) -> torch.Tensor:
    """Rows [g[e], g[e+1]) of the (optionally gathered) input times weight[e]; optional scatter of
    the output rows to ``permute_indices``; activation applied at the end."""
    rows = a.size(0) * topk if gather else a.size(0)
    c = torch.zeros(rows, weight.size(-1), dtype=a.dtype, device=a.device)
    g = group_indices.tolist()
    for e in range(weight.size(0)):
        lo, hi = g[e], g[e + 1]
        src = a[permute_indices[lo:hi] // topk] if gather else a[lo:hi]
        prod = src @ weight[e]
        if scatter:
            c[permute_indices[lo:hi]] = prod
        else:
            c[lo:hi] = prod
    return activation(c, act)


# --------------------------------------------------------------------------------------
# the layer -- src/moe_explore/functional/topk_moe.py:67-102
# --------------------------------------------------------------------------------------
def expert_compute(x: torch.Tensor, scores: torch.Tensor, indices: torch.Tensor, weight1: torch.Tensor,
                   weight2: torch.Tensor, act: str) -> torch.Tensor:
    """The per-expert loop of topk_moe_torch (topk_moe.py:80-102) with the in-place mul_ and
    scatter_reduce_ replaced by out-of-place multiply and index_add, so that autograd works.
    x [T,d]; scores [T,k]; indices int64 [T,k]; weight1 [E,d,2I or I]; weight2 [E,I,d] (in x's dtype, or a
    narrower one that is upcast per expert: lets a checker hold 16-bit weights and compute in fp32)."""
    topk = indices.size(1)
    num_experts = weight1.size(0)
    found = get_token_indices(indices, topk, num_experts, zero_prefix=True)
    g = found.group_indices.tolist()
    flat_scores = scores.reshape(-1, 1)
    out = torch.zeros_like(x)
    for e in range(num_experts):
        lo, hi = g[e], g[e + 1]
        if lo == hi:
            continue
        rows = found.indices[lo:hi]
        tok = rows // topk
        # weights stored in a narrower type than x are upcast one expert at a time (a no-op when the types agree)
        h = activation(x[tok] @ weight1[e].to(x.dtype), act)
        y = (h @ weight2[e].to(x.dtype)) * flat_scores[rows]
        out = out.index_add(0, tok, y)
    return out


def topk_moe(x: torch.Tensor, router_weight: torch.Tensor, weight1: torch.Tensor, weight2: torch.Tensor, topk: int,
             act: str, softmax_before_topk: bool = True, normalize_routing: bool = False) -> torch.Tensor:
    """topk_moe.py:67-102 end to end: router then the expert loop."""
    scores, indices = topk_router(x, router_weight, topk, softmax_before_topk, normalize_routing)
    return expert_compute(x, scores, indices, weight1, weight2, act)


def layer_fwd_bwd(x, scores, indices, weight1, weight2, act, grad_out):
    """Forward + torch.autograd backward of ``expert_compute``; returns out and the gradients
    with respect to x, scores, weight1, weight2 (all in the dtype of the inputs)."""
    x = x.detach().clone().requires_grad_(True)
    scores = scores.detach().clone().requires_grad_(True)
    weight1 = weight1.detach().clone().requires_grad_(True)
    weight2 = weight2.detach().clone().requires_grad_(True)
    out = expert_compute(x, scores, indices, weight1, weight2, act)
    out.backward(grad_out)
    return out.detach(), x.grad, scores.grad, weight1.grad, weight2.grad

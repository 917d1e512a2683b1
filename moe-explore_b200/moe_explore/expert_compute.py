"""The differentiable expert-compute step of the MoE layer on the native kernels.

forward : gate/up grouped GEMM with a fused GLU epilogue, its token rows either gathered by the GEMM's own
          operand loads (``gather_in_gemm``) or copied into the padded expert-sorted layout first -> down grouped
          GEMM -> weighted fold of the top-k slots (a separate deterministic kernel, or -- ``fused_combine``,
          forward-only -- scaled and added into the output by the down GEMM's epilogue).
backward: score-scaled gather of dOut (+ router-weight gradient as a row dot product) ->
          grouped GEMM against W2^T with the activation's derivative fused (GLU or plain) -> grouped GEMM against W1^T
          and an unweighted fold for dX -> two K-grouped GEMMs for the expert weight gradients.

The reference's forward is topk_moe_forward (src/moe_explore/functional/topk_moe.py:16-54);
it has no backward.  The gradients follow from out[t] = sum_s score[t,s] * (act(x_t W1[e]) W2[e]).
"""
from __future__ import annotations

import torch

from moe_explore import _native
from moe_explore.functional.activation import is_glu
from moe_explore.routing_plan import RoutingPlan


class ExpertCompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scores, weight1, weight2, plan: RoutingPlan, act: str, gather_in_gemm: bool, fused_combine: bool):
        _native.require_cuda(x, scores, weight1, weight2)
        assert x.dim() == 2 and weight1.dim() == 3 and weight2.dim() == 3
        T, d = x.shape
        E, d1, n1 = weight1.shape
        inter = weight2.size(1)
        assert d1 == d and weight2.size(0) == E and weight2.size(2) == d, "weight shapes do not match the input"
        assert n1 == (2 * inter if is_glu(act) else inter), "weight1 width does not match weight2 and the activation"
        assert plan.num_rows == T * plan.topk and plan.num_experts == E
        x = x.contiguous()
        scores = scores.to(x.dtype).contiguous()
        weight1 = weight1.contiguous()
        weight2 = weight2.contiguous()
        rp = plan.padded_rows
        new = lambda *shape: torch.empty(*shape, dtype=x.dtype, device=x.device)
        needs_grad = any(ctx.needs_input_grad[:4])

        hidden = new(rp, inter)
        # the un-activated product, needed by the backward pass (not kept for inference or without an activation)
        keep = act is not None and needs_grad
        pre_act = new(rp, n1) if (is_glu(act) or keep) else None
        if gather_in_gemm:
            xs = None
            _native.mgrouped_gemm_gather(x, plan.row_src, plan.topk, weight1, hidden, pre_act, plan.mtile_expert,
                                         plan.tile_pairs, plan.num_mtiles, rp, act, plan.status, rows=plan.num_rows)
        else:
            xs = new(rp, d)
            _native.dispatch_rows(x, plan.dst_row, plan.row_src, plan.num_mtiles, xs, plan.topk)
            _native.mgrouped_gemm(xs, weight1, hidden, pre_act, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, False,
                                  act, plan.status, rows=plan.num_rows)
        if fused_combine and not needs_grad:
            # forward only: the backward pass needs the per-slot rows for the router-weight gradient
            out = torch.zeros(T, d, dtype=x.dtype, device=x.device)
            _native.mgrouped_gemm_combine(hidden, weight2, out, plan.row_src, scores, plan.topk, plan.mtile_expert,
                                          plan.tile_pairs, plan.num_mtiles, False, plan.status, rows=plan.num_rows)
            return out
        ys = new(rp, d)
        _native.mgrouped_gemm(hidden, weight2, ys, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, False, None,
                              plan.status, rows=plan.num_rows)
        out = new(T, d)
        _native.combine_topk(ys, scores, plan.dst_row, out, plan.topk)

        ctx.plan = plan
        ctx.act = act
        ctx.gathered = bool(gather_in_gemm)
        ctx.save_for_backward(x if gather_in_gemm else xs, pre_act, hidden, ys, scores, weight1, weight2)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        xs, pre_act, hidden, ys, scores, weight1, weight2 = ctx.saved_tensors
        plan: RoutingPlan = ctx.plan
        act = ctx.act
        T, d = grad_out.shape
        rp = plan.padded_rows
        grad_out = grad_out.contiguous()
        new = lambda *shape: torch.empty(*shape, dtype=grad_out.dtype, device=grad_out.device)

        gs = new(rp, d)
        d_scores = torch.zeros(T, plan.topk, dtype=grad_out.dtype, device=grad_out.device)  # dropped slots keep 0
        _native.combine_bwd(grad_out, scores, ys, plan.row_src, plan.num_mtiles, gs, d_scores, plan.topk)
        d_pre = new(rp, weight1.size(2))
        if act is None:     # linear "activation": d_pre = gs @ W2^T
            _native.mgrouped_gemm(gs, weight2, d_pre, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, True, None,
                                  plan.status, rows=plan.num_rows)
        else:
            _native.mgrouped_gemm_dglu(gs, weight2, pre_act, d_pre, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, act,
                                       plan.status, rows=plan.num_rows)
        dxs = new(rp, d)
        _native.mgrouped_gemm(d_pre, weight1, dxs, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, True, None, plan.status,
                              rows=plan.num_rows)
        dx = new(T, d)
        _native.combine_topk(dxs, None, plan.dst_row, dx, plan.topk)
        d_w1 = torch.empty_like(weight1)
        if ctx.gathered:    # xs is the layer input in token order: its rows are gathered by the loads again
            _native.kgrouped_gemm_gather(xs, plan.row_src, plan.topk, d_pre, d_w1, plan.pad_offsets, plan.status,
                                         rows=plan.num_rows, tag="dw1")
        else:
            _native.kgrouped_gemm(xs, d_pre, d_w1, plan.pad_offsets, plan.status, rows=plan.num_rows, tag="dw1")
        d_w2 = torch.empty_like(weight2)
        _native.kgrouped_gemm(hidden, gs, d_w2, plan.pad_offsets, plan.status, rows=plan.num_rows, tag="dw2")
        return dx, d_scores, d_w1, d_w2, None, None, None, None


# Fusing the row gather into the gate/up GEMM's loads saves the copy of T*k rows into the expert-sorted layout
# (and, in training, keeps only the [T, d] input instead of the [R, d] copy for the weight1 gradient) -- but the 32
# four-row gather copies that replace one 128-row tile copy per stage cost ~95 cycles each on B200, which makes the
# gate/up GEMM 3.3x slower at the Mixtral shape (10.2 ms against 3.1 ms; the copy it saves takes 0.05 ms).  So the
# copy-first form is the default and the fused gather is for callers that are short of memory.
GATHER_IN_GEMM_DEFAULT = False


def expert_compute(x, scores, weight1, weight2, plan: RoutingPlan, act, gather_in_gemm=None,
                   fused_combine: bool = False) -> torch.Tensor:
    """out[t] = sum_s scores[t,s] * (act(x[t] @ weight1[e]) @ weight2[e]),  e = expert of (t, s).

    ``gather_in_gemm``: token rows are gathered by the gate/up GEMM's operand loads (tile::gather4) instead of being
    copied into the expert-sorted layout first (None = the package default).  ``fused_combine``: when no gradient
    is needed, the down GEMM's epilogue multiplies each row by its router weight and adds it into the output
    (vector reductions; the order of the k additions is not fixed, so the result is not bit-reproducible);
    ignored when a gradient is required."""
    if gather_in_gemm is None:
        gather_in_gemm = GATHER_IN_GEMM_DEFAULT
    return ExpertCompute.apply(x, scores, weight1, weight2, plan, None if act is None else str(act), bool(gather_in_gemm),
                               bool(fused_combine))

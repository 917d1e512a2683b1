"""Expert-parallel MoE layer: experts sharded over the ranks of one node, tokens stay data-parallel.

Rank g owns experts [g*E/G, (g+1)*E/G) -- their weights and weight gradients never move.  Per pass
there is one exchange each way (NCCL all-to-all over NVLink, uneven splits):

  forward : sort the local (token, slot) rows by global expert (= by owner rank, then by expert)
            -> exchange per-expert counts -> DISPATCH rows to their owners -> local grouped GEMMs
            -> COMBINE rows back -> weighted fold of the top-k slots at the source.
  backward: score-scaled dOut rows are dispatched the same way, the owners run the backward GEMMs
            (expert weight gradients stay local) and dX rows are combined back and folded.

The reference has no multi-GPU path; the single-GPU semantics it must reproduce are those of
topk_moe_forward (reference: src/moe_explore/functional/topk_moe.py:10-64).

The bookkeeping below is plain torch and device-agnostic; the row movement and the expert compute go
through an ``ops`` object.  ``NativeOps`` (the default, CUDA only) calls the library's kernels.  Tests
of the multi-rank logic on CPU ranks inject their own ``ops``; nothing in this module computes on
the CPU by itself.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from moe_explore import _native
from moe_explore.routing_plan import RoutingPlan, build_routing_plan


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class NativeOps:
    """Row movement and local expert compute on the library's CUDA kernels."""

    def sort_by_expert(self, flat_experts: torch.Tensor, num_experts: int):
        """-> (perm int64 [R], counts int64 [E]) with the stable counting sort."""
        plan = build_routing_plan(flat_experts, num_experts, 1, want_perm=True)
        counts = (plan.group_indices[1:] - plan.group_indices[:-1]).to(torch.int64)
        return plan.perm, counts

    def gather(self, src: torch.Tensor, index32: torch.Tensor, div: int) -> torch.Tensor:
        """out[r] = src[index32[r] // div]."""
        out = torch.empty(index32.numel(), src.size(1), dtype=src.dtype, device=src.device)
        if div != 1:
            index32 = torch.div(index32, div, rounding_mode="floor").to(torch.int32)
        _native.unpad_rows(src, index32, out)
        return out

    def fold(self, rows: torch.Tensor, scores: Optional[torch.Tensor], inv_perm32: torch.Tensor, num_tokens: int,
             topk: int) -> torch.Tensor:
        """out[t] = sum_s scores[t,s] * rows[inv_perm[t*topk+s]] (scores None = 1)."""
        out = torch.empty(num_tokens, rows.size(1), dtype=rows.dtype, device=rows.device)
        _native.combine_topk(rows, scores, inv_perm32, out, topk)
        return out

    def fold_bwd(self, grad_out, scores, rows_back, perm32_padded, tiles, topk):
        """g[r] = scores[perm[r]] * grad_out[perm[r] // topk]; dscores[j] = <grad_out[t], rows_back[inv_perm[j]]>."""
        g = torch.empty(perm32_padded.numel(), grad_out.size(1), dtype=grad_out.dtype, device=grad_out.device)
        dscores = torch.empty_like(scores)
        _native.combine_bwd(grad_out, scores, rows_back, perm32_padded, tiles, g, dscores, topk)
        return g, dscores

    def local_forward(self, recv_x, local_expert_ids, weight1, weight2, act):
        """Rows received for the local experts -> (y in received order, saved state)."""
        plan = build_routing_plan(local_expert_ids, weight1.size(0), 1, want_perm=False)
        rp, d = plan.padded_rows, recv_x.size(1)
        new = lambda *s: torch.empty(*s, dtype=recv_x.dtype, device=recv_x.device)
        xs = new(rp, d)
        _native.gather_rows(recv_x, plan.row_src, plan.num_mtiles, xs, 1)
        hidden = new(rp, weight2.size(1))
        pre_act = new(rp, weight1.size(2))
        _native.mgrouped_gemm(xs, weight1, hidden, pre_act, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, False, act, plan.status,
                              rows=plan.num_rows)
        ys = new(rp, d)
        _native.mgrouped_gemm(hidden, weight2, ys, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, False, None, plan.status,
                              rows=plan.num_rows)
        y = new(recv_x.size(0), d)
        _native.unpad_rows(ys, plan.dst_row, y)
        return y, (plan, xs, hidden, pre_act)

    def local_backward(self, recv_g, state, weight1, weight2, act):
        """-> (dx in received order, d_weight1, d_weight2)."""
        plan, xs, hidden, pre_act = state
        rp, d = plan.padded_rows, recv_g.size(1)
        new = lambda *s: torch.empty(*s, dtype=recv_g.dtype, device=recv_g.device)
        gs = new(rp, d)
        _native.gather_rows(recv_g, plan.row_src, plan.num_mtiles, gs, 1)
        d_pre = new(rp, pre_act.size(1))
        _native.mgrouped_gemm_dglu(gs, weight2, pre_act, d_pre, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, act, plan.status,
                                   rows=plan.num_rows)
        dxs = new(rp, d)
        _native.mgrouped_gemm(d_pre, weight1, dxs, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles, True, None, plan.status,
                              rows=plan.num_rows)
        d_w1 = torch.empty_like(weight1)
        _native.kgrouped_gemm(xs, d_pre, d_w1, plan.pad_offsets, plan.status, rows=plan.num_rows, tag="dw1")
        d_w2 = torch.empty_like(weight2)
        _native.kgrouped_gemm(hidden, gs, d_w2, plan.pad_offsets, plan.status, rows=plan.num_rows, tag="dw2")
        dx = new(recv_g.size(0), d)
        _native.unpad_rows(dxs, plan.dst_row, dx)
        return dx, d_w1, d_w2


@dataclass
class DispatchLayout:
    """Who sends how many rows to whom, for one routing decision."""
    perm: torch.Tensor               # int64 [R]: flat (token, slot) position of the r-th row in expert order
    inv_perm32: torch.Tensor         # int32 [R]: position in expert order of flat position j
    perm32_padded: torch.Tensor      # int32 [ceil(R/128)*128]: perm, padded with -1
    tiles: torch.Tensor              # int32 [1]: ceil(R/128)
    send_splits: list                # rows this rank sends to each rank
    recv_splits: list                # rows this rank receives from each rank
    local_expert_ids: torch.Tensor   # int64 [sum(recv_splits)]: local expert of each received row


def build_dispatch_layout(indices: torch.Tensor, num_experts: int, group, ops) -> DispatchLayout:
    """``indices`` int64 [T, topk] global expert ids.  One small all-to-all of per-expert counts and one
    host read of the split sizes (NCCL needs them on the host)."""
    world = dist.get_world_size(group)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    e_local = num_experts // world
    flat = indices.reshape(-1)
    R = flat.numel()
    perm, counts = ops.sort_by_expert(flat, num_experts)
    send_counts = counts.view(world, e_local).contiguous()
    recv_counts = torch.empty_like(send_counts)          # [source rank, local expert]
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    host = torch.stack((send_counts.sum(1), recv_counts.sum(1))).cpu()
    send_splits, recv_splits = host[0].tolist(), host[1].tolist()
    local_ids = torch.arange(e_local, device=flat.device).repeat(world)
    local_expert_ids = torch.repeat_interleave(local_ids, recv_counts.reshape(-1), output_size=sum(recv_splits))
    inv = torch.empty(R, dtype=torch.int32, device=flat.device)
    inv[perm] = torch.arange(R, dtype=torch.int32, device=flat.device)
    padded = torch.full((_round_up(max(R, 1), 128),), -1, dtype=torch.int32, device=flat.device)
    padded[:R] = perm.to(torch.int32)
    tiles = torch.full((1,), padded.numel() // 128, dtype=torch.int32, device=flat.device)
    return DispatchLayout(perm, inv, padded, tiles, send_splits, recv_splits, local_expert_ids)


def _exchange(rows: torch.Tensor, in_splits, out_splits, group) -> torch.Tensor:
    out = torch.empty(sum(out_splits), rows.size(1), dtype=rows.dtype, device=rows.device)
    with _native.timed("ep:all_to_all"):
        dist.all_to_all_single(out, rows, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out


class EPExpertCompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scores, weight1, weight2, layout: DispatchLayout, topk, act, group, ops):
        T = x.size(0)
        R = T * topk
        x = x.contiguous()
        scores = scores.to(x.dtype).contiguous()
        send_x = ops.gather(x, layout.perm32_padded[:R], topk)
        recv_x = _exchange(send_x, layout.send_splits, layout.recv_splits, group)       # dispatch
        y_recv, state = ops.local_forward(recv_x, layout.local_expert_ids, weight1, weight2, act)
        y_back = _exchange(y_recv, layout.recv_splits, layout.send_splits, group)       # combine
        out = ops.fold(y_back, scores, layout.inv_perm32, T, topk)
        ctx.layout, ctx.topk, ctx.act, ctx.group, ctx.ops, ctx.state = layout, topk, act, group, ops, state
        ctx.save_for_backward(scores, y_back, weight1, weight2)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        scores, y_back, weight1, weight2 = ctx.saved_tensors
        layout, topk, ops, group = ctx.layout, ctx.topk, ctx.ops, ctx.group
        T = grad_out.size(0)
        R = T * topk
        grad_out = grad_out.contiguous()
        y_pad = y_back
        if y_back.size(0) != layout.perm32_padded.numel():
            y_pad = torch.zeros(layout.perm32_padded.numel(), y_back.size(1), dtype=y_back.dtype, device=y_back.device)
            y_pad[:R] = y_back
        # y_back row r belongs to flat position perm[r]: fold_bwd reads rows_back[r] for padded row r
        g_send, d_scores = ops.fold_bwd(grad_out, scores, y_pad, layout.perm32_padded, layout.tiles, topk)
        g_recv = _exchange(g_send[:R], layout.send_splits, layout.recv_splits, group)   # dispatch gradients
        dx_recv, d_w1, d_w2 = ops.local_backward(g_recv, ctx.state, weight1, weight2, ctx.act)
        dx_back = _exchange(dx_recv, layout.recv_splits, layout.send_splits, group)     # combine gradients
        dx = ops.fold(dx_back, None, layout.inv_perm32, T, topk)
        return dx, d_scores, d_w1, d_w2, None, None, None, None, None


def ep_expert_compute(x: torch.Tensor, scores: torch.Tensor, indices: torch.Tensor, local_weight1: torch.Tensor,
                      local_weight2: torch.Tensor, num_experts: int, act: str = "swiglu", group=None,
                      ops=None) -> torch.Tensor:
    """Expert-parallel ``out[t] = sum_s scores[t,s] * expert_{indices[t,s]}(x[t])``.

    x [T, d] (this rank's tokens), scores [T, k], indices int64 [T, k] with GLOBAL expert ids,
    local_weight1 [E/G, d, 2I], local_weight2 [E/G, I, d] (this rank's experts).  Differentiable with
    respect to x, scores and the local weights."""
    if ops is None:
        _native.require_cuda(x, scores, indices, local_weight1, local_weight2)
        ops = NativeOps()
    group = group if group is not None else dist.group.WORLD
    with _native.timed("ep:layout"):
        layout = build_dispatch_layout(indices, num_experts, group, ops)
    return EPExpertCompute.apply(x, scores, local_weight1.contiguous(), local_weight2.contiguous(), layout,
                                 indices.size(1), str(act), group, ops)

"""Expert-parallel MoE layer: experts sharded over the ranks of one node, tokens stay data-parallel.

Rank g owns experts [g*E/G, (g+1)*E/G) -- their weights and weight gradients never move.  Per pass
there is one exchange each way:

  forward : sort the local (token, slot) rows by global expert (= by owner rank, then by expert)
            -> exchange per-expert counts -> DISPATCH rows to their owners -> local grouped GEMMs
            -> COMBINE rows back -> weighted fold of the top-k slots at the source.
  backward: score-scaled dOut rows are dispatched the same way, the owners run the backward GEMMs
            (expert weight gradients stay local) and dX rows are combined back and folded.

Two data paths implement the exchanges:

  * peer mode (``EPContext``; the fast path): token rows never go through a collective.  Every rank
    publishes its tokens in a peer-mapped (symmetric-memory) buffer; the expert owners PULL the rows
    they need straight into the padded expert-sorted layout with the library's gather kernel (loads
    over NVLink), and the down-projection / dX grouped GEMMs PUSH every output row into the token
    owner's buffer from their epilogue (stores over NVLink, overlapped with the next tile's math).
    Only row metadata (8 bytes per routed row) and three tiny barriers go through NCCL.  A variant of the
    dispatch (``EPContext(..., dispatch="dma")``) keeps the SMs out of it: every rank sorts its rows by destination
    expert into a peer-mapped send buffer, and the owners fetch each (expert, source rank) block -- contiguous on
    both sides -- with one asynchronous memcpy on the copy engines.
  * collective mode: rows are exchanged with ``all_to_all_single`` (NCCL) before and after the local
    GEMMs; kept as the baseline the peer path is measured against.

The reference has no multi-GPU path; the single-GPU semantics it must reproduce are those of
topk_moe_forward (reference: src/moe_explore/functional/topk_moe.py:10-64).

The bookkeeping below is plain torch and device-agnostic; the row movement and the expert compute go
through an ``ops`` object.  ``NativeOps`` (the default, CUDA only) calls the library's kernels.  Tests
of the multi-rank logic on CPU ranks inject their own ``ops``; nothing in this module computes on
the CPU by itself.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple, Optional

import torch
import torch.distributed as dist

from moe_explore import _native
from moe_explore.routing_plan import RoutingPlan, _report, build_routing_plan, device_status


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def balanced_placement(expert_load, world: int) -> torch.Tensor:
    """Static expert placement that evens out the routed rows per rank.

    ``expert_load``: per-expert row counts (any 1-D sequence / tensor of length E, e.g. measured over a
    few steps).  Every rank still owns exactly E / world experts.  Returns ``remap`` (int64 [E]):
    ``remap[e]`` is the position of logical expert e in the sharded weight tensors, i.e. rank
    ``remap[e] // (E / world)`` owns it.  Apply it to the router's indices (``remap[indices]``) and store
    expert e's weights at position ``remap[e]``.

    Greedy longest-processing-time assignment with a per-rank capacity: experts in decreasing load order,
    each to the least-loaded rank that still has a free slot; inside a rank the positions go by increasing load."""
    load = [float(v) for v in (expert_load.tolist() if hasattr(expert_load, "tolist") else expert_load)]
    num_experts = len(load)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    cap = num_experts // world
    total = [0.0] * world
    owned = [[] for _ in range(world)]
    for e in sorted(range(num_experts), key=lambda i: (-load[i], i)):
        r = min((g for g in range(world) if len(owned[g]) < cap), key=lambda g: (total[g], g))
        owned[r].append(e)
        total[r] += load[e]
    remap = [0] * num_experts
    for r in range(world):
        # within a rank: lightest expert first.  The expert-parallel pipeline starts its GEMMs as soon as the rows of
        # the first experts have arrived, so the first slice should be small, and a hot expert (under a Zipf router one
        # expert can hold 40 % of a rank's rows) should come last, when there is earlier work to hide its pull under.
        for slot, e in enumerate(sorted(owned[r], key=lambda i: (load[i], i))):
            remap[e] = r * cap + slot
    return torch.tensor(remap, dtype=torch.int64)


def pipeline_schedule(rows_per_expert, first_fraction: float = 1.0 / 32, growth: float = 2.0, max_slices: int = 8):
    """Slices [begin, end) of the local expert list, in launch order, for pipelining the pull of slice c+1 against the
    GEMMs of slice c.  The pulls run back to back from the start of the pass, so slice c can start computing when a
    fraction f_c of all rows has arrived; with pulls P and GEMMs G per pass (P < G) nothing waits after the first
    slice as long as every slice holds at most G/P times the rows before it.  Hence: a first slice of about
    ``first_fraction`` of the rows (its pull is the only one nothing hides), then slices of at most ``growth`` times
    the rows already scheduled -- cut by ROWS, which under a skewed router is far from cutting by expert count."""
    rows = [int(v) for v in rows_per_expert]
    n, total = len(rows), sum(rows)
    if n <= 1 or total == 0:
        return [(0, n)]
    slices, begin, done = [], 0, 0
    target = max(total * first_fraction, 1.0)
    for e in range(n - 1):
        done += rows[e]
        if done >= target and len(slices) < max_slices - 1:
            slices.append((begin, e + 1))
            begin = e + 1
            target = done * (1.0 + growth)
    slices.append((begin, n))
    return slices


def pair_rows(rows_per_expert):
    """Rows of every entry of the list of row-tile pairs the routing metadata builds for these per-expert row counts:
    an expert with r rows has ceil(r / 128) tiles and ceil(tiles / 2) pairs of (at most) 256 rows."""
    out = []
    for r in rows_per_expert:
        r = int(r)
        pairs = ((r + 127) // 128 + 1) // 2
        out.extend(min(256, r - 256 * p) for p in range(pairs))
    return out


class Slice(NamedTuple):
    """One slice of a pass's pipeline: a range of the local expert list, or of the list of row-tile pairs."""
    experts: tuple
    pairs: tuple
    rows: float


class NativeOps:
    """Row movement and local expert compute on the library's CUDA kernels."""

    def status_word(self, device) -> torch.Tensor:
        """The device status word the kernels report into (read together with the split sizes, once per step)."""
        return device_status(device)

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
    status = ops.status_word(flat.device).to(torch.int64) if hasattr(ops, "status_word") else torch.zeros(1, dtype=torch.int64, device=flat.device)
    host = _native.read_small(torch.cat((send_counts.sum(1), recv_counts.sum(1), status)))   # the one host read of the step
    _report(int(host[-1]))                                                                   # e.g. an expert id out of range
    send_splits, recv_splits = host[:world], host[world:2 * world]
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


# --------------------------------------------------------------------------------------------------
# peer mode: pull dispatch / push combine over peer-mapped memory
# --------------------------------------------------------------------------------------------------
class EPContext:
    """Peer-mapped buffers of one expert-parallel layer on one rank (created collectively).

    ``src`` [T, d] holds this rank's tokens (forward) or upstream gradient rows (backward) for the
    expert owners to pull; ``y_back`` / ``dx_back`` [ceil(T*topk/128)*128, d] receive the rows the
    owners push back, in this rank's expert-sorted order.  A context serves one forward/backward pair
    at a time: ``y_back`` is read again by the backward pass."""

    def __init__(self, group, num_tokens: int, hidden: int, topk: int, dtype, device, allocate=True, dispatch="pull"):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_tokens, self.hidden, self.topk, self.dtype, self.device = num_tokens, hidden, topk, dtype, device
        self.rows_up = _round_up(max(num_tokens * topk, 1), 128)
        self.busy = False
        # "pull": the owners' pull kernels read token rows from `src`; "dma": every rank sorts its rows by destination
        # expert into `send` and the owners copy whole (expert, source) blocks with the copy engines
        assert dispatch in ("pull", "dma")
        self.dispatch = dispatch
        self.chunks = 8          # equal slices of the local expert list, used when `geometric` is off
        self.geometric = True    # slices cut by received rows, small first and growing (pipeline_schedule)
        # ... in the list of row-tile pairs, so that a slice may end inside an expert: True / False, or None = only when
        # slices of whole experts would leave more than `hot_slice_fraction` of the rows to one slice
        self.slice_pairs = None
        self.hot_slice_fraction = 0.85
        self.comm_stream = None  # side stream the pulls run on (created with the buffers)
        # SMs the grouped GEMMs leave free while rows are pulled from peers (read by the native ops): a pull CTA
        # that shares an SM with a GEMM CTA gets almost none of the SM's L2 ingress (measured at 2 ranks: 37.8 ms
        # of pull kernels per step with every SM busy, 14.1 ms with 8 SMs free, the GEMMs no slower since they
        # are power-limited).  Nothing to gain with one rank: local rows arrive fast either way.
        self.reserved_sms = 8 if self.world > 1 else 0
        # How rows are pulled: "ldst" = the load/store kernel spread over all SMs (it also runs, slowly, on the SMs that
        # run GEMM CTAs -- and slows those GEMMs), "dedicated" = the same kernel as one 1024-thread CTA on each reserved
        # SM (it cannot share an SM with a GEMM CTA either way), "bulk" = the copy-engine kernel, one CTA on each
        # reserved SM.  Measured at 2 ranks with 8 reserved SMs: 12.6 ms of pulls per step with "ldst", 29.5 ms with
        # "bulk" (15.1 ms with 16 SMs): a warp of the bulk kernel has one row in flight at a time.
        self.pull_mode = "ldst"
        if allocate:
            self._allocate_symmetric()

    def _allocate_symmetric(self):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm

        def make(rows):
            t = symm.empty(rows, self.hidden, dtype=self.dtype, device=self.device)
            handle = symm.rendezvous(t, self.group)
            ptrs = torch.tensor(list(handle.buffer_ptrs), dtype=torch.int64, device=self.device)
            return t, handle, ptrs

        self.src, self._h_src, self.src_ptrs = make(self.num_tokens)
        if self.dispatch == "dma":
            self.send, self._h_send, self.send_ptrs = make(self.rows_up)
            self.send_addresses = [int(p) for p in self._h_send.buffer_ptrs]   # host copy of the peers' base addresses
        self.y_back, self._h_y, self.y_ptrs = make(self.rows_up)
        self.dx_back, self._h_dx, self.dx_ptrs = make(self.rows_up)
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.comm_stream = torch.cuda.Stream(device=self.device)


@dataclass
class PeerLayout:
    """Routing bookkeeping of one step in peer mode (all tensors on the compute device)."""
    perm32_padded: torch.Tensor   # int32 [rows_up]: flat position of the r-th row in expert order, -1 padding
    inv_perm32: torch.Tensor      # int32 [R]
    tiles: torch.Tensor           # int32 [1]: rows_up / 128
    plan: object                  # local routing plan over the received rows (padded expert-sorted layout)
    p_rank: torch.Tensor          # int32 [RP]: rank that owns the token of padded row p (-1 padding)
    p_tok: torch.Tensor           # int32 [RP]: token index on that rank
    p_dest: torch.Tensor          # int32 [RP]: row of that rank's y_back / dx_back this row is pushed to
    p_scale: torch.Tensor         # fp32  [RP]: router weight of the row (applied to dOut rows in backward)
    num_received: int
    expert_rows: list = None      # rows received per local expert (host list; drives the pipeline schedule)
    counts: list = None           # "dma" dispatch: counts[s][g] rows rank s routes to global expert position g (host)


def build_peer_layout(indices: torch.Tensor, scores: torch.Tensor, num_experts: int, group, ops, after_sort=None,
                      want_counts: bool = False) -> PeerLayout:
    """Exchange the row metadata of one routing decision: an all-gather of per-expert counts, one host
    read of the split sizes, and an all-to-all of (token index, router weight) per routed row.
    ``after_sort(perm)`` runs right after the local sort and BEFORE the collectives (which then order whatever it
    enqueued ahead of every peer's later reads); ``want_counts`` also brings the full [ranks, experts] count table to
    the host."""
    world, me = dist.get_world_size(group), dist.get_rank(group)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    e_local = num_experts // world
    topk = indices.size(1)
    flat = indices.reshape(-1)
    R, dev = flat.numel(), flat.device
    perm, counts = ops.sort_by_expert(flat, num_experts)
    if after_sort is not None:
        after_sort(perm)
    gathered = torch.empty(world * num_experts, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(gathered, counts.contiguous(), group=group)
    all_counts = gathered.view(world, num_experts)
    pair = all_counts.view(world, world, e_local).sum(-1)              # [source, owner] rows
    status = ops.status_word(dev).to(torch.int64) if hasattr(ops, "status_word") else torch.zeros(1, dtype=torch.int64, device=dev)
    local_rows = all_counts[:, me * e_local:(me + 1) * e_local].sum(0)       # rows each local expert receives
    parts = (pair.reshape(-1), local_rows, all_counts.reshape(-1), status) if want_counts else (pair.reshape(-1), local_rows, status)
    host_all = _native.read_small(torch.cat(parts))                        # the one host read of the step
    _report(int(host_all[-1]))                                             # e.g. an expert id out of range
    send_splits = host_all[me * world:(me + 1) * world]
    recv_splits = host_all[me:world * world:world]
    expert_rows = host_all[world * world:world * world + e_local]
    host_counts = None
    if want_counts:
        base = world * world + e_local
        host_counts = [host_all[base + s * num_experts: base + (s + 1) * num_experts] for s in range(world)]
    num_received = sum(recv_splits)
    send_base = pair.cumsum(1) - pair                                   # start of each owner's segment at the source
    base_on_source = send_base[:, me]                                   # [world]
    recv_counts = pair[:, me]
    recv_offsets = recv_counts.cumsum(0) - recv_counts

    meta_send = torch.empty(R, 2, dtype=torch.int32, device=dev)
    meta_send[:, 0] = torch.div(perm, topk, rounding_mode="floor")
    meta_send[:, 1] = scores.reshape(-1)[perm].float().view(torch.int32)
    meta_recv = torch.empty(num_received, 2, dtype=torch.int32, device=dev)
    dist.all_to_all_single(meta_recv, meta_send, output_split_sizes=recv_splits, input_split_sizes=send_splits,
                           group=group)

    ranks = torch.arange(world, device=dev)
    src_rank = torch.repeat_interleave(ranks, recv_counts, output_size=num_received)
    local_ids = torch.arange(e_local, device=dev).repeat(world)
    local_expert = torch.repeat_interleave(local_ids, all_counts[:, me * e_local:(me + 1) * e_local].reshape(-1),
                                           output_size=num_received)
    dest_row = base_on_source[src_rank] + (torch.arange(num_received, device=dev) - recv_offsets[src_rank])

    plan = ops.local_plan(local_expert, e_local)
    valid = plan.row_src >= 0
    j = plan.row_src.clamp_min(0).long()
    if num_received == 0:
        src_rank = torch.zeros(1, dtype=torch.int64, device=dev)
        dest_row = torch.zeros(1, dtype=torch.int64, device=dev)
        meta_recv = torch.zeros(1, 2, dtype=torch.int32, device=dev)
    minus1 = torch.full((), -1, dtype=torch.int32, device=dev)
    p_rank = torch.where(valid, src_rank[j].to(torch.int32), minus1)
    p_tok = torch.where(valid, meta_recv[j, 0], minus1)
    p_dest = torch.where(valid, dest_row[j].to(torch.int32), minus1)
    p_scale = torch.where(valid, meta_recv[j, 1].view(torch.float32), torch.zeros((), device=dev))

    inv = torch.empty(R, dtype=torch.int32, device=dev)
    inv[perm] = torch.arange(R, dtype=torch.int32, device=dev)
    padded = torch.full((_round_up(max(R, 1), 128),), -1, dtype=torch.int32, device=dev)
    padded[:R] = perm.to(torch.int32)
    tiles = torch.full((1,), padded.numel() // 128, dtype=torch.int32, device=dev)
    return PeerLayout(padded, inv, tiles, plan, p_rank.contiguous(), p_tok.contiguous(), p_dest.contiguous(),
                      p_scale.contiguous(), num_received, expert_rows, host_counts)


class NativePeerOps(NativeOps):
    """Peer-mode data path on the library's kernels (CUDA only)."""

    def local_plan(self, local_expert_ids, num_local_experts):
        return build_routing_plan(local_expert_ids, num_local_experts, 1, want_perm=False)

    def publish(self, ctx: EPContext, rows: torch.Tensor):
        # An element-wise kernel, not a memcpy: a device-to-device memcpy may be queued on a copy engine behind a long
        # host transfer of another stream (a training loop that uploads the next batch while this step runs), and
        # everything after the publish waits for it.
        with _native.timed("ep:publish"):
            torch.mul(rows, 1, out=ctx.src)

    def barrier(self, ctx: EPContext):
        """Stream-ordered: every rank's work enqueued so far is complete before any rank continues."""
        with _native.timed("ep:barrier"):
            dist.all_reduce(ctx._flag, group=ctx.group)

    def fold_bwd_scores(self, grad_out, scores, y_back, perm32_padded, tiles, topk):
        dscores = torch.empty_like(scores)
        _native.combine_bwd(grad_out, scores, y_back, perm32_padded, tiles, None, dscores, topk)
        return dscores

    @staticmethod
    def _chunks(ctx: EPContext, lay: PeerLayout):
        """Pipeline schedule: slices [begin, end) of the local expert list, in launch order.  By default they are cut
        by the rows each local expert received (``pipeline_schedule``); ``ctx.geometric = False`` cuts ``ctx.chunks``
        slices of equal expert count instead."""
        experts = lay.plan.num_experts
        if ctx.geometric and lay.expert_rows is not None and len(lay.expert_rows) == experts:
            return pipeline_schedule(lay.expert_rows)
        n = max(1, min(ctx.chunks, experts))
        return [(experts * c // n, experts * (c + 1) // n) for c in range(n) if experts * (c + 1) // n > experts * c // n]

    @classmethod
    def _slices(cls, ctx: EPContext, lay: PeerLayout):
        """The pipeline slices of a pass, in launch order.  With the pull dispatch and known per-expert row counts they
        are cut in the list of row-tile pairs, so that a slice may end inside an expert: under a skewed router one
        expert can hold most of a rank's rows (93 % on the hottest rank of 8 with Zipf(1.1) popularity), and slices of
        whole experts then leave its pull with nothing to hide behind.  (Measured on 8 GPUs the step came out the same
        either way, 78-80 ms: the GEMMs that run beside the pulls lose what the pulls take, whichever they are.  The
        pair ranges keep the GEMM stream from ever waiting on one huge pull.)  ``ctx.slice_pairs``: True / False force the
        choice, None (default) cuts inside experts only when whole experts would give one slice more than
        ``ctx.hot_slice_fraction`` of the rows.  Otherwise: whole experts (``_chunks``)."""
        experts = lay.plan.num_experts
        whole = [Slice(chunk, (0, 0), cls._slice_rows(lay, chunk)) for chunk in cls._chunks(ctx, lay)]
        if (ctx.dispatch == "pull" and ctx.geometric and ctx.slice_pairs is not False and lay.expert_rows is not None
                and len(lay.expert_rows) == experts):
            total = max(float(sum(lay.expert_rows)), 1.0)
            # (measured at 2 ranks, where whole experts leave 72 % to the last slice: cutting inside experts costs 1.5 %
            # -- more of the GEMM work then runs beside a pull, on fewer SMs -- so it is done only where it is needed)
            if ctx.slice_pairs or max(s.rows for s in whole) > ctx.hot_slice_fraction * total:
                rows = pair_rows(lay.expert_rows)
                if len(rows) > 1:
                    return [Slice((0, 0), (lo, hi), float(sum(rows[lo:hi]))) for lo, hi in pipeline_schedule(rows)]
        return whole

    @staticmethod
    def _slice_rows(lay: PeerLayout, experts):
        if lay.expert_rows is None:
            return lay.num_received * (experts[1] - experts[0]) / max(lay.plan.num_experts, 1)
        return sum(lay.expert_rows[experts[0]:experts[1]])

    @staticmethod
    def _sm_count(ctx: EPContext) -> int:
        return _native.query_device(ctx.device.index if ctx.device.index is not None else torch.cuda.current_device())[0]

    @classmethod
    def _gemm_options(cls, ctx: EPContext, piece: Slice, last: bool):
        """Launch options of one pipeline slice: its experts or pairs, and ``ctx.reserved_sms`` SMs left free for the
        pulls of the slices after it (the last slice has no pull beside it and takes every SM; so does every slice
        when the copy engines do the dispatch)."""
        reserve = ctx.reserved_sms > 0 and not last and ctx.dispatch != "dma"
        cap = max(cls._sm_count(ctx) - ctx.reserved_sms, 2) if reserve else 0
        return _native.gemm_options(max_ctas=cap, experts=piece.experts, pairs=piece.pairs)

    def sort_into_send(self, ctx: EPContext, rows: torch.Tensor, perm: torch.Tensor, scores=None):
        """ctx.send[r] = rows[perm[r] // topk] (times scores.flat[perm[r]] when given): this rank's rows in expert
        order, i.e. grouped by destination, for the owners' block copies."""
        R = perm.numel()
        tok = torch.full((ctx.rows_up,), -1, dtype=torch.int32, device=rows.device)
        tok[:R] = torch.div(perm, ctx.topk, rounding_mode="floor").to(torch.int32)
        rank0 = torch.where(tok >= 0, 0, -1).to(torch.int32)
        scale = None
        if scores is not None:
            scale = torch.zeros(ctx.rows_up, dtype=torch.float32, device=rows.device)
            scale[:R] = scores.reshape(-1)[perm].float()
        # (filled by kernels with scalar arguments: a host-to-device memcpy of a few bytes would queue on a copy
        # engine behind any large upload another stream has in flight)
        base = torch.full((1,), rows.data_ptr(), dtype=torch.int64, device=rows.device)
        tiles = torch.zeros(4, dtype=torch.int32, device=rows.device)
        tiles[0] = ctx.rows_up // 128
        with _native.timed("ep:sort_into_send"):
            _native.gather_rows_peer(base, rank0, tok, scale, tiles, ctx.send)
        ctx._send_keepalive = (rows, base)   # the kernel reads them asynchronously

    def _dma_chunks(self, ctx: EPContext, lay: PeerLayout, dst):
        """Generator over the pipeline slices: each ``next()`` enqueues, on the side stream, the block copies that
        fill one slice of ``dst`` (padded expert-sorted rows) from every rank's send buffer and yields the event
        recorded after them.  (A generator, so that the caller can enqueue the copies of slice c+1 and then launch the
        GEMMs of slice c: issuing a few hundred memcpys takes the host milliseconds, which must not hold up the
        GPU.)  Expert e of this rank receives counts[s][g] rows from rank s (g = its global position); they start at
        the sum of counts[s][:g] in that rank's send buffer and, here, after the rows of the ranks before s inside
        the expert's padded segment."""
        plan, chunks = lay.plan, self._chunks(ctx, lay)
        world, me, counts = ctx.world, ctx.rank, lay.counts
        e_local = plan.num_experts
        row_bytes = ctx.hidden * dst.element_size()
        first = me * e_local
        send_offset = [sum(counts[s][:first]) for s in range(world)]   # first row of my experts in rank s's send buffer
        main = torch.cuda.current_stream()
        ctx.comm_stream.wait_stream(main)
        with torch.cuda.stream(ctx.comm_stream):
            _native.zero_padding_rows(plan.row_src, plan.num_mtiles, dst)
        # Every copy goes to the one side stream.  (Spreading a slice's copies over four streams, to engage more than one
        # copy engine, ended in a cross-rank stall between the copies and the next stream-ordered barrier on a
        # two-GPU run -- NCCL's watchdog ended it -- so it is not done.)
        pad_row = 0
        for lo, hi in chunks:
            d_addr, s_addr, sizes = [], [], []
            for e in range(lo, hi):
                g = first + e
                row = pad_row
                for s in range(world):
                    n = counts[s][g]
                    if n:
                        d_addr.append(dst.data_ptr() + row * row_bytes)
                        s_addr.append(ctx.send_addresses[s] + send_offset[s] * row_bytes)
                        sizes.append(n * row_bytes)
                        row += n
                        send_offset[s] += n
                pad_row += (row - pad_row + 127) // 128 * 128
            with torch.cuda.stream(ctx.comm_stream):
                _native.copy_blocks(d_addr, s_addr, sizes)
                ev = torch.cuda.Event()
                ev.record(ctx.comm_stream)
            yield ev

    def _pull_chunks(self, ctx: EPContext, lay: PeerLayout, scale, dst):
        """Enqueue the pull of every slice on the side stream; returns one event per slice."""
        plan, chunks = lay.plan, self._slices(ctx, lay)
        main = torch.cuda.current_stream()
        ctx.comm_stream.wait_stream(main)          # the layout arrays and the destination exist
        # copy-engine pull: one CTA per reserved SM while GEMMs hold the others; every SM when nothing is reserved
        bulk_ctas = dedicated_ctas = 0
        if ctx.pull_mode == "bulk":
            bulk_ctas = ctx.reserved_sms if ctx.reserved_sms > 0 else self._sm_count(ctx)
        elif ctx.pull_mode == "dedicated":
            dedicated_ctas = ctx.reserved_sms if ctx.reserved_sms > 0 else self._sm_count(ctx)
        events = []
        with torch.cuda.stream(ctx.comm_stream):
            for chunk in chunks:
                _native.gather_rows_peer(ctx.src_ptrs, lay.p_rank, lay.p_tok, scale, plan.num_mtiles, dst,
                                         plan.tile_pairs, plan.num_experts, bulk_ctas=bulk_ctas, status=plan.status,
                                         experts=chunk.experts if chunk.pairs[1] <= chunk.pairs[0] else None,
                                         pairs=chunk.pairs, dedicated_ctas=dedicated_ctas)
                ev = torch.cuda.Event()
                ev.record(ctx.comm_stream)
                events.append(ev)
        return events

    def peer_forward(self, ctx: EPContext, lay: PeerLayout, weight1, weight2, act):
        """Dispatch (pull) chunk c+1 on the side stream while the gate/up and down GEMMs of chunk c run; the
        down GEMM's epilogue pushes its rows to the token owners (combine)."""
        plan, chunks = lay.plan, self._slices(ctx, lay)
        rp, d = plan.padded_rows, ctx.hidden
        new = lambda *s: torch.empty(*s, dtype=ctx.dtype, device=ctx.device)
        xs, hidden, pre_act = new(rp, d), new(rp, weight2.size(1)), new(rp, weight1.size(2))
        main = torch.cuda.current_stream()
        events = self._dma_chunks(ctx, lay, xs) if ctx.dispatch == "dma" else iter(self._pull_chunks(ctx, lay, None, xs))
        ahead = next(events)
        for chunk in chunks:
            event, ahead = ahead, next(events, None)     # the next slice's rows are on their way before this one computes
            with _native.timed("ep:wait_pull"):
                main.wait_event(event)
            opts, rows = self._gemm_options(ctx, chunk, chunk is chunks[-1]), chunk.rows
            _native.mgrouped_gemm(xs, weight1, hidden, pre_act, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles,
                                  False, act, plan.status, rows=rows, options=opts)
            _native.mgrouped_gemm_push(hidden, weight2, ctx.y_ptrs, lay.p_rank, lay.p_dest, plan.mtile_expert,
                                       plan.tile_pairs, plan.num_mtiles, False, plan.status, rows=rows, options=opts)
        return xs, hidden, pre_act

    def peer_backward(self, ctx: EPContext, lay: PeerLayout, state, weight1, weight2, act):
        xs, hidden, pre_act = state
        plan, chunks = lay.plan, self._slices(ctx, lay)
        rp, d = plan.padded_rows, ctx.hidden
        new = lambda *s: torch.empty(*s, dtype=ctx.dtype, device=ctx.device)
        gs, d_pre = new(rp, d), new(rp, pre_act.size(1))
        main = torch.cuda.current_stream()
        # score-scaled dOut rows: scaled by the owner's pull kernel, or already by the source ("dma" dispatch)
        events = self._dma_chunks(ctx, lay, gs) if ctx.dispatch == "dma" else iter(self._pull_chunks(ctx, lay, lay.p_scale, gs))
        ahead = next(events)
        for chunk in chunks:
            event, ahead = ahead, next(events, None)
            with _native.timed("ep:wait_pull"):
                main.wait_event(event)
            opts, rows = self._gemm_options(ctx, chunk, chunk is chunks[-1]), chunk.rows
            _native.mgrouped_gemm_dglu(gs, weight2, pre_act, d_pre, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles,
                                       act, plan.status, rows=rows, options=opts)
            _native.mgrouped_gemm_push(d_pre, weight1, ctx.dx_ptrs, lay.p_rank, lay.p_dest, plan.mtile_expert,
                                       plan.tile_pairs, plan.num_mtiles, True, plan.status, rows=rows, options=opts)
        # no pull runs beside the weight-gradient GEMMs: they use every SM
        d_w1 = torch.empty_like(weight1)
        _native.kgrouped_gemm(xs, d_pre, d_w1, plan.pad_offsets, plan.status, rows=lay.num_received, tag="dw1")
        d_w2 = torch.empty_like(weight2)
        _native.kgrouped_gemm(hidden, gs, d_w2, plan.pad_offsets, plan.status, rows=lay.num_received, tag="dw2")
        return d_w1, d_w2


class PeerEPExpertCompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scores, weight1, weight2, indices, num_experts, act, ep: EPContext, ops):
        T, topk = x.size(0), indices.size(1)
        assert T == ep.num_tokens and topk == ep.topk and x.size(1) == ep.hidden, "context was built for another shape"
        if ep.busy:
            raise RuntimeError("this EPContext still holds the rows of a forward pass whose backward has not run")
        scores = scores.to(x.dtype).contiguous()
        x = x.contiguous()
        dma = getattr(ep, "dispatch", "pull") == "dma"
        if not dma:
            ops.publish(ep, x)
        with _native.timed("ep:layout"):
            # its collectives follow the publish (or the sort into the send buffer) and so order it before peers' reads
            lay = build_peer_layout(indices, scores, num_experts, ep.group, ops,
                                    after_sort=(lambda perm: ops.sort_into_send(ep, x, perm)) if dma else None,
                                    want_counts=dma)
        state = ops.peer_forward(ep, lay, weight1, weight2, act)
        ops.barrier(ep)                                                          # every owner has pushed its rows
        out = ops.fold(ep.y_back, scores, lay.inv_perm32, T, topk)
        ctx.ep, ctx.ops, ctx.lay, ctx.state, ctx.act = ep, ops, lay, state, act
        ctx.save_for_backward(scores, weight1, weight2)
        ep.busy = any(ctx.needs_input_grad)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        scores, weight1, weight2 = ctx.saved_tensors
        ep, ops, lay = ctx.ep, ctx.ops, ctx.lay
        T, topk = grad_out.size(0), ep.topk
        grad_out = grad_out.contiguous()
        d_scores = ops.fold_bwd_scores(grad_out, scores, ep.y_back, lay.perm32_padded, lay.tiles, topk)
        if getattr(ep, "dispatch", "pull") == "dma":
            R = T * topk
            ops.sort_into_send(ep, grad_out, lay.perm32_padded[:R].long(), scores)   # score-scaled, in expert order
        else:
            ops.publish(ep, grad_out)
        ops.barrier(ep)                                                          # every rank's dOut is in place
        d_w1, d_w2 = ops.peer_backward(ep, lay, ctx.state, weight1, weight2, ctx.act)
        ops.barrier(ep)                                                          # every owner has pushed its dX rows
        dx = ops.fold(ep.dx_back, None, lay.inv_perm32, T, topk)
        ep.busy = False
        return dx, d_scores, d_w1, d_w2, None, None, None, None, None


def ep_expert_compute(x: torch.Tensor, scores: torch.Tensor, indices: torch.Tensor, local_weight1: torch.Tensor,
                      local_weight2: torch.Tensor, num_experts: int, act: str = "swiglu", group=None,
                      ops=None, context: Optional[EPContext] = None) -> torch.Tensor:
    """Expert-parallel ``out[t] = sum_s scores[t,s] * expert_{indices[t,s]}(x[t])``.

    x [T, d] (this rank's tokens), scores [T, k], indices int64 [T, k] with GLOBAL expert ids,
    local_weight1 [E/G, d, 2I], local_weight2 [E/G, I, d] (this rank's experts).  Differentiable with
    respect to x, scores and the local weights.  With ``context`` (an ``EPContext`` built once for the
    layer) rows move over peer-mapped memory inside the gather kernel and the GEMM epilogues;
    without it they are exchanged with NCCL all-to-all collectives."""
    group = group if group is not None else (context.group if context is not None else dist.group.WORLD)
    if context is not None:
        if ops is None:
            _native.require_cuda(x, scores, indices, local_weight1, local_weight2)
            ops = NativePeerOps()
        return PeerEPExpertCompute.apply(x, scores, local_weight1.contiguous(), local_weight2.contiguous(), indices,
                                         num_experts, str(act), context, ops)
    if ops is None:
        _native.require_cuda(x, scores, indices, local_weight1, local_weight2)
        ops = NativeOps()
    with _native.timed("ep:layout"):
        layout = build_dispatch_layout(indices, num_experts, group, ops)
    return EPExpertCompute.apply(x, scores, local_weight1.contiguous(), local_weight2.contiguous(), layout,
                                 indices.size(1), str(act), group, ops)

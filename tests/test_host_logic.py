"""Host-side pieces that need no GPU: parameter bundles, the activation enum, router dispatch,
weight interleaving, and the differentiable torch cross-check of the layer."""
import math

import pytest
import torch

from moe_explore.functional.activation import Activation, activation
from moe_explore.functional.topk_moe import topk_moe_torch
from moe_explore.params import (ErnieRouterParams, GLUParams, MLPParams, MOEParams, RouterParams, TopkRouterParams,
                                interleave_gate_up)
from moe_explore.router import router
from oracle import moe_oracle as O


def test_dataclasses_keep_the_reference_field_order():
    w = torch.zeros(2, 4, 8)
    mlp = MLPParams(w, w, "swiglu")
    assert (mlp.weight1 is w) and mlp.activation == "swiglu"
    r = TopkRouterParams(torch.zeros(4, 2), 2)
    assert r.softmax_before_topk is True and r.normalize_routing is False
    p = MOEParams(r, mlp, 2, 2)
    assert p.shared_expert_params is None and p.num_experts == 2 and p.topk == 2
    g = GLUParams(w, w, w, Activation.SWIGLU)
    assert g.activation == "swiglu"


def test_activation_enum_and_errors():
    x = torch.randn(3, 8)
    assert torch.equal(activation(x, Activation.SWIGLU), O.activation(x, "swiglu"))
    assert torch.equal(activation(x, "geglu"), O.activation(x, "geglu"))
    assert torch.equal(activation(x, "silu"), O.activation(x, "silu"))
    assert torch.equal(activation(x, "gelu"), O.activation(x, "gelu"))
    with pytest.raises(AssertionError):
        activation(x, "relu")
    with pytest.raises(AssertionError):
        activation(torch.randn(3, 7), "swiglu")


def test_router_dispatch_and_values():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(10, 16, generator=g)
    wr = torch.randn(16, 6, generator=g)
    for sb in (True, False):
        for nm in (True, False):
            s, i = router(x, TopkRouterParams(wr, 2, sb, nm))
            so, io = O.topk_router(x, wr, 2, sb, nm)
            assert torch.equal(i, io) and torch.equal(s, so)
    bias = torch.randn(6, generator=g)
    s, i = router(x, ErnieRouterParams(wr, bias, 2))
    so, io = O.ernie_router(x, wr, bias, 2)
    assert torch.equal(i, io) and torch.equal(s, so)
    with pytest.raises(ValueError, match="Unsupported router type"):
        router(x, RouterParams())


def test_interleave_gate_up():
    gate = torch.arange(24.).reshape(2, 3, 4)
    up = -gate
    w = interleave_gate_up(gate, up)
    assert w.shape == (2, 3, 8)
    assert torch.equal(w[..., 0::2], gate) and torch.equal(w[..., 1::2], up)


def test_torch_cross_check_matches_oracle_and_is_differentiable():
    g = torch.Generator().manual_seed(1)
    T, d, E, k, I = 32, 16, 4, 2, 8
    x = torch.randn(T, d, generator=g, requires_grad=True)
    wr = (torch.randn(d, E, generator=g) * 0.1).requires_grad_(True)
    w1 = (torch.randn(E, d, 2 * I, generator=g) * 0.1).requires_grad_(True)
    w2 = (torch.randn(E, I, d, generator=g) * 0.1).requires_grad_(True)
    params = MOEParams(TopkRouterParams(wr, k, False, False), MLPParams(w1, w2, "swiglu"), E, k)
    out = topk_moe_torch(x, params)
    ref = O.topk_moe(x, wr, w1, w2, k, "swiglu", False, False)
    torch.testing.assert_close(out, ref)
    out.sum().backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in (x, wr, w1, w2))


@pytest.mark.parametrize("experts", [1, 5, 31, 32, 33, 64, 100, 128, 1000])
def test_pipeline_schedule_partitions_the_local_experts(experts):
    """The slices of a pipeline schedule tile [0, E) in launch order, without gaps, overlaps or empty slices -- cut by
    rows (the default), or into equal expert counts."""
    from types import SimpleNamespace

    from moe_explore.expert_parallel import NativePeerOps

    g = torch.Generator().manual_seed(experts)
    rows = torch.randint(0, 2000, (experts,), generator=g).tolist()
    for ctx, expert_rows in ((SimpleNamespace(chunks=8, geometric=True), rows), (SimpleNamespace(chunks=8, geometric=False), rows),
                             (SimpleNamespace(chunks=3, geometric=False), None), (SimpleNamespace(chunks=8, geometric=True), None)):
        lay = SimpleNamespace(plan=SimpleNamespace(num_experts=experts), expert_rows=expert_rows, num_received=sum(rows))
        schedule = NativePeerOps._chunks(ctx, lay)
        covered = 0
        for lo, hi in schedule:
            assert lo == covered and hi > lo
            covered = hi
        assert covered == experts and len(schedule) <= 8


def test_pipeline_schedule_is_cut_by_rows_not_by_expert_count():
    """Under a skewed router the first slice must stay small and no slice may hold more than `growth` times the rows
    scheduled before it (the condition under which only the first pull is exposed), unless a single expert is that
    big by itself."""
    from moe_explore.expert_parallel import balanced_placement, pipeline_schedule

    g = torch.Generator().manual_seed(1)
    E, world = 256, 4
    p = (torch.arange(1, E + 1, dtype=torch.float64) ** -1.1)[torch.randperm(E, generator=g)]
    u = torch.rand(32768, E, generator=g, dtype=torch.float64).clamp_min(1e-20)
    idx = torch.topk(torch.log(p / p.sum()) - torch.log(-torch.log(u)), 8, dim=-1).indices
    load = torch.bincount(idx.reshape(-1), minlength=E)
    remap = balanced_placement(load, world)
    e_local = E // world
    for r in range(world):
        # rows of the local experts in position order: ascending load inside a rank, the hot expert last
        local = torch.zeros(e_local, dtype=torch.int64)
        mine = (remap // e_local) == r
        local[(remap[mine] % e_local)] = load[mine]
        rows = local.tolist()
        assert rows == sorted(rows)
        total = sum(rows)
        schedule = pipeline_schedule(rows)
        assert schedule[0][0] == 0 and schedule[-1][1] == e_local
        first = sum(rows[schedule[0][0]:schedule[0][1]])
        assert first <= total / 32 + max(rows[:schedule[0][1]])          # about 1/32 of the rows, one expert of slack
        done = first
        for lo, hi in schedule[1:]:
            here = sum(rows[lo:hi])
            assert here <= 2.0 * done + rows[hi - 1] or hi - lo == 1 or (lo, hi) == schedule[-1]
            done += here
        assert done == total
    assert pipeline_schedule([0, 0, 0]) == [(0, 3)] and pipeline_schedule([5]) == [(0, 1)]
    assert pipeline_schedule([100] * 64, first_fraction=1 / 32) [0] == (0, 2)


def test_pipeline_slices_may_end_inside_a_hot_expert():
    """With the pull dispatch the slices are ranges of the list of row-tile pairs: they cover every pair once, the
    first one is small, and an expert that holds nearly all rows is cut into several slices instead of being the
    whole last one."""
    from types import SimpleNamespace

    from moe_explore.expert_parallel import NativePeerOps, pair_rows

    assert pair_rows([0, 1, 128, 129, 256, 257, 600]) == [1, 128, 129, 256, 256, 1, 256, 256, 88]
    rows = [40, 0, 130, 300, 500, 900, 1200, 258000]            # 31 light experts' worth and one hot one, roughly
    ctx = SimpleNamespace(dispatch="pull", geometric=True, slice_pairs=None, hot_slice_fraction=0.85, chunks=8)
    lay = SimpleNamespace(plan=SimpleNamespace(num_experts=len(rows)), expert_rows=rows, num_received=sum(rows))
    slices = NativePeerOps._slices(ctx, lay)
    per_pair = pair_rows(rows)
    assert slices[0].pairs[0] == 0 and slices[-1].pairs[1] == len(per_pair)
    for a, b in zip(slices, slices[1:]):
        assert a.pairs[1] == b.pairs[0] and a.pairs[1] > a.pairs[0]
    assert abs(sum(s.rows for s in slices) - sum(rows)) < 1e-6
    assert slices[0].rows <= sum(rows) / 32 + 256
    assert len(slices) >= 4 and slices[-1].rows < 0.75 * sum(rows)      # whole experts would end with a 98 % slice
    # whole-expert slices when asked for, when the copy engines do the dispatch, or when no expert dominates
    ctx.slice_pairs = False
    assert all(s.pairs == (0, 0) for s in NativePeerOps._slices(ctx, lay))
    ctx.slice_pairs, ctx.dispatch = True, "dma"
    assert all(s.pairs == (0, 0) for s in NativePeerOps._slices(ctx, lay))
    ctx.slice_pairs, ctx.dispatch = None, "pull"
    even = SimpleNamespace(plan=SimpleNamespace(num_experts=32), expert_rows=[1000 + 10 * i for i in range(32)], num_received=0)
    assert all(s.pairs == (0, 0) for s in NativePeerOps._slices(ctx, even))
    ctx.slice_pairs = True
    assert all(s.experts == (0, 0) for s in NativePeerOps._slices(ctx, even))


def test_status_codes_map_to_errors_and_warnings():
    """The Python view of a device status word: 0 is fine, the wave barrier's fall-back is a warning (the launch's
    results are valid), everything else raises."""
    import warnings

    from moe_explore import _native
    from moe_explore.routing_plan import _report

    assert _report(0) == 0
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        assert _report(_native.STATUS_WAVE_FALLBACK) == 4
    assert len(seen) == 1 and "wave barrier" in str(seen[0].message)
    for code, text in ((_native.STATUS_BAD_EXPERT_ID, "outside"), (_native.STATUS_BAD_LAYOUT, "does not describe"),
                       (2, "bounded wait")):
        with pytest.raises(_native.MoeNativeError, match=text):
            _report(code)


def test_options_struct_matches_the_library(native):
    import ctypes

    assert native.load().moe_gemm_options_size() == ctypes.sizeof(native.GemmOptions) == 56
    o = native.gemm_options(max_ctas=140, wave_sync=-1, wave_workers=3)
    assert (o.max_ctas, o.wave_sync, o.wave_workers, o.group_m, o.align_experts, o.single_cta, o.separate_copies,
            o.lane_stores, o.expert_begin, o.expert_end, o.pair_begin, o.pair_end, o.wave_counter) == (
        140, -1, 3, 0, 0, 0, 0, 0, 0, 0, 0, 0, None)


def test_oracle_upcasts_narrower_weights_per_expert():
    """The checker may hold 16-bit weights and compute in fp32: same result as upcasting everything first."""
    import torch

    from oracle import moe_oracle as O

    g = torch.Generator().manual_seed(0)
    x = torch.randn(40, 32, generator=g)
    w1 = (torch.randn(4, 32, 48, generator=g) * 0.1).bfloat16()
    w2 = (torch.randn(4, 24, 32, generator=g) * 0.1).bfloat16()
    top, idx = torch.topk(torch.randn(40, 4, generator=g), 2, dim=-1)
    s = torch.softmax(top, -1)
    a = O.expert_compute(x, s, idx, w1, w2, "swiglu")
    b = O.expert_compute(x, s, idx, w1.float(), w2.float(), "swiglu")
    assert torch.equal(a, b)


def test_harness_routings_and_tolerance_rule():
    """The harness helpers (routing generators, group cuts, tolerance rule) on the CPU: shapes, value ranges and the
    properties their names promise."""
    import torch

    from moe_explore import testing as H

    dev, dt = torch.device("cpu"), torch.float32
    torch.manual_seed(0)
    s, i = H.perfect_routing(64, 8, 2, dev, dt)
    assert s.shape == (64, 2) and i.shape == (64, 2)
    assert torch.bincount(i.reshape(-1), minlength=8).tolist() == [16] * 8
    s, i = H.random_routing(100, 16, 4, dev, dt)
    assert i.dtype == torch.int64 and int(i.min()) >= 0 and int(i.max()) < 16
    assert all(len(set(row)) == 4 for row in i.tolist())                    # k distinct experts per token
    s, i = H.random_skewed_routing(4000, 16, 2, num_skewed_experts=2, skew_factor=8, device=dev, dtype=dt)
    counts = torch.bincount(i.reshape(-1), minlength=16).float()
    top2 = counts.sort(descending=True).values[:2].sum()
    assert top2 > 0.4 * counts.sum()                                        # two experts draw 16 of 30 weight units
    p = H.zipf_popularity(64, 1.5, torch.Generator().manual_seed(1))
    assert abs(float(p.sum()) - 1.0) < 1e-5 and float(p.max() / p.min()) > 400
    s, i = H.popularity_routing(500, p, 8, dev, dt)
    assert all(len(set(row)) == 8 for row in i.tolist())
    g = H.random_groups(1000, 7, dev)
    assert g.dtype == torch.int32 and g[0] == 0 and g[-1] == 1000 and bool((g[1:] > g[:-1]).all())
    w = H.uniform_weight_init((4, 32, 64), dev, dt)
    assert float(w.abs().max()) <= math.sqrt(3) * math.sqrt(2 / 96) + 1e-6
    mlp = H.random_mlp(4, 32, 48, "swiglu", dev, dt)
    assert mlp.weight1.shape == (4, 32, 96) and mlp.weight2.shape == (4, 48, 32)
    a = torch.ones(8, 256, dtype=torch.bfloat16)
    atol, rtol = H.tolerances(a, a)
    assert atol == min(1e-2, 256 * 1.0 * 0.0078125 * 1e-2) and abs(rtol - 16 * 0.0078125 * 0.1) < 1e-12
    H.assert_close(a, a)
    with pytest.raises(AssertionError):
        H.assert_close(a, a * 1.5)

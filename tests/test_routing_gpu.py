"""Routing metadata kernels against the oracle: integer work, compared bit for bit."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _plan(idx, E, k):
    from moe_explore.routing_plan import build_routing_plan

    plan = build_routing_plan(idx.cuda(), E, k)
    torch.cuda.synchronize()
    return plan


def _check_against_oracle(idx, E):
    k = idx.size(1)
    plan = _plan(idx, E, k)
    ref = O.get_token_indices(idx.cpu(), k, E, zero_prefix=True)
    assert torch.equal(plan.group_indices.cpu(), ref.group_indices)
    assert plan.perm.dtype == torch.int64 and torch.equal(plan.perm.cpu(), ref.indices)
    po, row_src, dst_row, mte = O.padded_layout(idx.cpu(), E)
    n, num_pairs, bound_written, _ = plan.num_mtiles.tolist()
    assert bound_written == plan.mtile_expert.numel()
    assert n == int(po[-1]) // 128
    # tile pairs: every tile appears exactly once, both tiles of a pair belong to the same expert
    pairs = plan.tile_pairs[:num_pairs].cpu().tolist()
    seen = []
    for info in pairs:
        first, expert, second = info & 0xFFFFF, (info >> 20) & 0x7FF, (info >> 31) & 1
        assert expert == int(mte[first])
        seen.append(first)
        if second:
            assert int(mte[first]) == int(mte[first + 1])
            seen.append(first + 1)
        else:
            assert first + 1 == n or int(mte[first + 1]) != int(mte[first])
    assert seen == list(range(n))
    # the per-expert exclusive prefix of pair counts follows the pair list
    bound = plan.mtile_expert.numel()
    prefix = plan.tile_pairs[bound: bound + E + 1].cpu().tolist()
    per_expert = [(int(po[e + 1]) - int(po[e])) // 128 for e in range(E)]
    expect = [0]
    for t in per_expert:
        expect.append(expect[-1] + (t + 1) // 2)
    assert prefix == expect and prefix[-1] == num_pairs
    # the host's view of the pair list (what the expert-parallel pipeline cuts its slices in) is the device's:
    # as many entries, and for every pair the rows of the tiles it covers
    from moe_explore.expert_parallel import pair_rows

    counts = torch.bincount(idx.reshape(-1).cpu(), minlength=E).tolist()
    host_pairs = pair_rows(counts)
    assert len(host_pairs) == num_pairs
    live = (row_src >= 0).view(-1, 128).sum(1).tolist()                   # routed rows of every tile in use
    assert host_pairs == [live[info & 0xFFFFF] + (live[(info & 0xFFFFF) + 1] if (info >> 31) & 1 else 0) for info in pairs]
    assert torch.equal(plan.pad_offsets.cpu(), po)
    assert torch.equal(plan.row_src[: n * 128].cpu(), row_src)
    assert torch.equal(plan.dst_row.cpu(), dst_row)
    assert torch.equal(plan.mtile_expert[:n].cpu(), mte)
    assert int(plan.status.item()) == 0
    plan.check()
    return plan


@pytest.mark.parametrize("case", ["uniform", "empty_experts", "one_expert", "single_row", "many_experts"])
def test_golden_id_patterns(case, native):
    z = load_golden("token_indices")
    idx = torch.from_numpy(z[case + "_idx"])
    E = int(z[case + "_E"])
    plan = _check_against_oracle(idx, E)
    # the reference's own outputs: group boundaries exact, each expert's segment the same set of rows
    assert torch.equal(plan.group_indices.cpu(), torch.from_numpy(z[case + "_group_zero_prefix"]))
    ref_perm = torch.from_numpy(z[case + "_ref_perm"])
    g = plan.group_indices.cpu().tolist()
    mine = plan.perm.cpu()
    for e in range(E):
        assert torch.equal(torch.sort(mine[g[e]:g[e + 1]]).values, torch.sort(ref_perm[g[e]:g[e + 1]]).values)


@pytest.mark.parametrize("T,E,k", [(5, 8, 2), (128, 8, 2), (999, 64, 8), (2011, 64, 8), (1025, 3, 1), (4096, 256, 8),
                                   (16384, 60, 4), (8192, 8, 2), (777, 1, 1), (300, 1024, 4)])
def test_random_routing(T, E, k, native):
    g = torch.Generator().manual_seed(T + E)
    idx = torch.topk(torch.randn(T, E, generator=g), k, dim=-1, sorted=False).indices
    _check_against_oracle(idx, E)


def test_public_get_token_indices(native):
    from moe_explore.expert_permute import get_token_indices

    g = torch.Generator().manual_seed(3)
    idx = torch.topk(torch.randn(700, 16, generator=g), 4, dim=-1, sorted=False).indices
    for zero_prefix in (True, False):
        got = get_token_indices(idx.cuda(), 4, 16, zero_prefix=zero_prefix)
        ref = O.get_token_indices(idx, 4, 16, zero_prefix=zero_prefix)
        assert got.group_indices.dtype == ref.group_indices.dtype
        assert torch.equal(got.group_indices.cpu(), ref.group_indices)
        assert torch.equal(got.indices.cpu(), ref.indices)


@pytest.mark.parametrize("dist", ["normal", "zipf", "degenerate"])
@pytest.mark.parametrize("T", [128, 1024, 8192, 65536])
def test_routing_stress_sweep(T, dist, native):
    """d=2048-layer routing of the stress sweep: E=64, top-8, three router distributions, up to R=524288."""
    E, k = 64, 8
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(T, E, generator=g)
    if dist == "zipf":
        p = torch.arange(1, E + 1, dtype=torch.float32) ** -1.5
        p = p[torch.randperm(E, generator=g)]
        u = torch.rand(T, E, generator=g).clamp_min(1e-20)
        logits = torch.log(p / p.sum()) - torch.log(-torch.log(u))
    elif dist == "degenerate":
        hot = torch.rand(T, generator=g) < 0.95
        logits[hot, 5] += 20.0
        logits[:, 40:48] = -1e4
    idx = torch.topk(logits, k, dim=-1, sorted=False).indices
    plan = _check_against_oracle(idx, E)
    if dist == "degenerate":
        counts = (plan.group_indices[1:] - plan.group_indices[:-1]).cpu()
        assert int((counts[40:48] == 0).all()) == 1 and int(counts[5]) >= 0.9 * T


def test_out_of_range_ids_are_flagged_not_placed(native):
    from moe_explore._native import MoeNativeError

    idx = torch.tensor([[0, 1], [9, 2], [3, -1]], dtype=torch.int64)
    plan = _plan(idx, 4, 2)
    assert plan.group_indices.cpu().tolist() == [0, 1, 2, 3, 4]
    assert int(plan.status.item()) == 100
    # dropped positions are marked, not left undefined: no padded row, and the tail of the permutation is -1
    assert plan.dst_row.cpu().tolist()[2] == -1 and plan.dst_row.cpu().tolist()[5] == -1
    assert plan.perm.cpu().tolist()[4:] == [-1, -1] and sorted(plan.perm.cpu().tolist()[:4]) == [0, 1, 3, 4]
    with pytest.raises(MoeNativeError, match="outside"):
        plan.check()
    assert int(plan.status.item()) == 0   # reading the word clears it


def test_layer_with_an_out_of_range_id_stays_in_bounds(native):
    """One bad expert id in a whole forward + backward: the status word says so, the (token, slot) pairs with the bad
    id contribute nothing, every other output equals the layer run on the valid pairs alone, and every index a kernel
    consumed was either a valid row or the -1 marker (checked on the host)."""
    from moe_explore._native import MoeNativeError
    from moe_explore.expert_compute import expert_compute
    from moe_explore.routing_plan import build_routing_plan

    T, d, E, k, I = 300, 128, 8, 2, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g, device="cuda") * std).bfloat16()
    x, w1, w2, grad = mk(T, d), mk(E, d, 2 * I, std=0.05), mk(E, I, d, std=0.05), mk(T, d)
    idx = torch.topk(torch.randn(T, E, generator=g, device="cuda"), k, dim=-1, sorted=False).indices
    scores = torch.softmax(torch.randn(T, k, generator=g, device="cuda"), -1).bfloat16()
    bad = idx.clone()
    bad[17, 1] = E + 3          # out of range
    bad[101, 0] = -2            # negative
    for gather_in_gemm in (False, True):
        leaves = [t.detach().clone().requires_grad_() for t in (x, scores, w1, w2)]
        plan = build_routing_plan(bad, E, k)
        out = expert_compute(*leaves, plan, "swiglu", gather_in_gemm=gather_in_gemm)
        out.backward(grad)
        torch.cuda.synchronize()
        assert int(plan.status.item()) == 100
        rp = plan.padded_rows
        dst, src, perm = plan.dst_row.cpu(), plan.row_src.cpu(), plan.perm.cpu()
        assert ((dst == -1) | ((dst >= 0) & (dst < rp))).all() and int((dst == -1).sum()) == 2
        assert ((src == -1) | ((src >= 0) & (src < T * k)))[: int(plan.num_mtiles[0]) * 128].all()
        assert ((perm == -1) | ((perm >= 0) & (perm < T * k))).all() and int((perm == -1).sum()) == 2
        with pytest.raises(MoeNativeError, match="outside"):
            plan.check()
        # reference: the same layer with the two bad slots given weight zero and any valid expert
        ok_idx = bad.clone()
        ok_idx[17, 1] = 0
        ok_idx[101, 0] = 0
        ok_scores = scores.float().clone()
        ok_scores[17, 1] = 0
        ok_scores[101, 0] = 0
        ref = O.layer_fwd_bwd(x.float(), ok_scores, ok_idx, w1.float(), w2.float(), "swiglu", grad.float())
        rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert out.isfinite().all() and rel(out, ref[0]) <= 2e-2
        assert rel(leaves[0].grad, ref[1]) <= 2e-2 and rel(leaves[2].grad, ref[3]) <= 2e-2 and rel(leaves[3].grad, ref[4]) <= 2e-2
        ds = leaves[1].grad.float()
        assert float(ds[17, 1]) == 0.0 and float(ds[101, 0]) == 0.0
        mask = torch.ones(T, k, dtype=torch.bool, device="cuda")
        mask[17, 1] = mask[101, 0] = False
        assert rel(ds[mask], ref[2][mask]) <= 2e-2


def test_group_prefix_that_is_not_a_prefix_is_reported(native):
    """plan_from_groups with a prefix that does not end at the row count (or is not monotone): status 5, the
    offending rows get no padded row, nothing is written out of bounds."""
    from moe_explore._native import MoeNativeError
    from moe_explore.routing_plan import plan_from_groups

    for groups in ([0, 40, 100, 90], [0, 40, 100, 130], [5, 40, 100, 128]):
        plan = plan_from_groups(torch.tensor(groups, dtype=torch.int32, device="cuda"), 128)
        torch.cuda.synchronize()
        assert int(plan.status.item()) == 5
        dst = plan.dst_row.cpu()
        assert ((dst == -1) | ((dst >= 0) & (dst < plan.padded_rows))).all()
        with pytest.raises(MoeNativeError, match="does not describe"):
            plan.check()


def test_empty_input(native):
    plan = _plan(torch.zeros(0, 2, dtype=torch.int64), 8, 2)
    assert plan.group_indices.cpu().tolist() == [0] * 9
    assert plan.num_mtiles.tolist()[:2] == [0, 0]

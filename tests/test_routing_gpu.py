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
    n, num_pairs = plan.num_mtiles.tolist()
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
    with pytest.raises(MoeNativeError, match="outside"):
        plan.check()


def test_empty_input(native):
    plan = _plan(torch.zeros(0, 2, dtype=torch.int64), 8, 2)
    assert plan.group_indices.cpu().tolist() == [0] * 9
    assert plan.num_mtiles.tolist() == [0, 0]

"""The oracle against the committed outputs of the reference implementation (tests/golden/*.npz,
produced by tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import moe_oracle as O

LAYER_CASES = ["layer_small_swiglu", "layer_small_geglu_norm", "layer_small_silu", "layer_small_gelu"]


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _same_segments(perm_a, perm_b, group):
    g = group.tolist()
    for e in range(len(g) - 1):
        a = torch.sort(perm_a[g[e]:g[e + 1]]).values
        b = torch.sort(perm_b[g[e]:g[e + 1]]).values
        if not torch.equal(a, b):
            return False
    return True


def _redraw_inputs(seed, T, d, E, I, glu):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g)
    wr = torch.randn(d, E, generator=g) * 0.02
    w1 = torch.randn(E, d, 2 * I if glu else I, generator=g) * 0.02
    w2 = torch.randn(E, I, d, generator=g) * 0.02
    return x, wr, w1, w2


def _checksum(*tensors):
    return np.array([float(t.double().sum()) for t in tensors] + [float(t.double().abs().sum()) for t in tensors])


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_matches_reference(name):
    z = load_golden(name)
    seed, T, d, E, k, I, sb, nm = [int(v) for v in z["meta"]]
    act = str(z["act"])
    x, wr, w1, w2 = _t(z["x"]), _t(z["router_weight"]), _t(z["weight1"]), _t(z["weight2"])
    scores, idx = O.topk_router(x, wr, k, bool(sb), bool(nm))
    assert torch.equal(idx, _t(z["indices"]))                      # integer: bit-exact
    assert torch.equal(scores, _t(z["scores"]))                    # same torch ops: bit-exact
    zp = O.get_token_indices(idx, k, E, zero_prefix=True)
    inc = O.get_token_indices(idx, k, E, zero_prefix=False)
    assert zp.group_indices.dtype == torch.int32 and torch.equal(zp.group_indices, _t(z["group_zero_prefix"]))
    assert torch.equal(inc.group_indices, _t(z["group_inclusive"]).to(inc.group_indices.dtype))
    assert _same_segments(zp.indices, _t(z["ref_perm"]), zp.group_indices)
    out = O.expert_compute(x, scores, idx, w1, w2, act)
    # fp32: the reference accumulates with scatter_reduce_, the oracle with index_add -- same values, summation order may differ
    torch.testing.assert_close(out, _t(z["out"]), rtol=1e-5, atol=1e-6)
    out2 = O.topk_moe(x, wr, w1, w2, k, act, bool(sb), bool(nm))
    assert torch.equal(out, out2)


def test_first_benchmark_config_matches_reference():
    """T=512 d=256 E=8 top-2 I=512 fp32 seed 0: inputs are re-drawn from the seed."""
    z = load_golden("layer_c1")
    seed, T, d, E, k, I, sb, nm = [int(v) for v in z["meta"]]
    x, wr, w1, w2 = _redraw_inputs(seed, T, d, E, I, True)
    if not np.allclose(_checksum(x, wr, w1, w2), z["input_checksum"], rtol=1e-9):
        pytest.skip("torch's CPU generator produced different inputs than when the fixture was made")
    scores, idx = O.topk_router(x, wr, k, bool(sb), bool(nm))
    assert torch.equal(idx, _t(z["indices"]))
    torch.testing.assert_close(scores, _t(z["scores"]), rtol=1e-6, atol=1e-7)
    out = O.expert_compute(x, scores, idx, w1, w2, str(z["act"]))
    torch.testing.assert_close(out, _t(z["out"]), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("case", ["uniform", "empty_experts", "one_expert", "single_row", "many_experts"])
def test_token_indices_match_reference(case):
    z = load_golden("token_indices")
    idx = _t(z[case + "_idx"])
    E = int(z[case + "_E"])
    k = idx.size(1)
    zp = O.get_token_indices(idx, k, E, zero_prefix=True)
    inc = O.get_token_indices(idx, k, E, zero_prefix=False)
    assert torch.equal(zp.group_indices, _t(z[case + "_group_zero_prefix"]))
    assert torch.equal(inc.group_indices, _t(z[case + "_group_inclusive"]).to(inc.group_indices.dtype))
    assert _same_segments(zp.indices, _t(z[case + "_ref_perm"]), zp.group_indices)
    # the canonical order is the stable one
    flat = idx.reshape(-1)
    assert torch.equal(flat[zp.indices], torch.sort(flat).values)
    for e in range(E):
        seg = zp.indices[int(zp.group_indices[e]): int(zp.group_indices[e + 1])]
        assert torch.equal(seg, torch.sort(seg).values)


def test_padded_layout_is_consistent():
    z = load_golden("token_indices")
    for case in ["uniform", "empty_experts", "one_expert", "single_row", "many_experts"]:
        idx = _t(z[case + "_idx"])
        E = int(z[case + "_E"])
        po, row_src, dst_row, mte = O.padded_layout(idx, E)
        assert int(po[-1]) % 128 == 0 and row_src.numel() == int(po[-1])
        assert torch.equal(row_src[dst_row.long()], torch.arange(idx.numel(), dtype=torch.int32))
        assert int((row_src >= 0).sum()) == idx.numel()
        flat = idx.reshape(-1)
        valid = row_src >= 0
        rows = torch.nonzero(valid).squeeze(1)
        assert torch.equal(flat[row_src[rows].long()].to(torch.int32), mte[(rows // 128)])


def test_activations_and_reduce_match_reference():
    z = load_golden("activations")
    x = _t(z["x"])
    for name in ("silu", "gelu", "swiglu", "geglu"):
        assert torch.equal(O.activation(x, name), _t(z[name])), name
    assert torch.equal(O.scale_and_reduce(_t(z["y"]), _t(z["s"]), 6, 4), _t(z["scale_and_reduce"]))


def test_routers_match_reference():
    z = load_golden("routers")
    x, wr, bias = _t(z["x"]), _t(z["router_weight"]), _t(z["bias"])
    for sb in (False, True):
        for nm in (False, True):
            sc, ix = O.topk_router(x, wr, 3, sb, nm)
            assert torch.equal(ix, _t(z[f"topk_sb{int(sb)}_nm{int(nm)}_indices"]))
            assert torch.equal(sc, _t(z[f"topk_sb{int(sb)}_nm{int(nm)}_scores"]))
    sc, ix = O.ernie_router(x, wr, bias, 3)
    assert torch.equal(ix, _t(z["ernie_indices"])) and torch.equal(sc, _t(z["ernie_scores"]))


def test_oracle_gradients_by_finite_differences():
    """No reference backward exists; the oracle's autograd is checked numerically in float64."""
    g = torch.Generator().manual_seed(5)
    T, d, E, k, I = 6, 8, 3, 2, 4
    x = torch.randn(T, d, generator=g, dtype=torch.float64, requires_grad=True)
    w1 = (torch.randn(E, d, 2 * I, generator=g, dtype=torch.float64) * 0.5).requires_grad_(True)
    w2 = (torch.randn(E, I, d, generator=g, dtype=torch.float64) * 0.5).requires_grad_(True)
    scores = torch.rand(T, k, generator=g, dtype=torch.float64, requires_grad=True)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    assert torch.autograd.gradcheck(lambda a, s, b, c: O.expert_compute(a, s, idx, b, c, "swiglu"), (x, scores, w1, w2),
                                    eps=1e-6, atol=1e-5)

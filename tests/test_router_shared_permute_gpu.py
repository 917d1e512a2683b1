"""The steps either side of the expert GEMMs: the opt-in fused router kernel, the shared-expert branch and the
stand-alone permute API, each against torch / the oracle on the GPU."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-2


def relerr(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("softmax_before,normalize", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("T,E,k,dtype", [(1000, 8, 2, torch.bfloat16), (513, 60, 4, torch.bfloat16), (300, 64, 8, torch.float16),
                                          (257, 256, 8, torch.float32), (64, 1024, 8, torch.float32), (5, 8, 8, torch.float32)])
def test_fused_router_kernel_on_tie_free_logits(T, E, k, dtype, softmax_before, normalize, native):
    """Logits without ties (a random permutation of distinct values per row): the kernel selects exactly torch.topk's
    experts -- in descending order of value, which is torch.topk(sorted=True)'s order -- and its scores match the
    reference's torch ops (router.py:17-35) to a rounding of the output type; the histogram equals bincount."""
    g = torch.Generator(device="cuda").manual_seed(T + E)
    # distinct, exactly representable values: multiples of 1/8 in [-E/16, E/16), shuffled per row
    base = (torch.arange(E, device="cuda", dtype=torch.float32) - E // 2) / 8
    logits = torch.stack([base[torch.randperm(E, generator=g, device="cuda")] for _ in range(T)]).to(dtype)
    scores, idx, counts = native.router_topk(logits, k, softmax_before, normalize, want_counts=True)
    ref_in = torch.softmax(logits, -1, dtype=torch.float32) if softmax_before else logits
    ref_s, ref_i = torch.topk(ref_in, k, dim=-1, sorted=True)
    if not softmax_before:
        ref_s = torch.softmax(ref_s, -1, dtype=torch.float32)
    if normalize:
        ref_s = ref_s / ref_s.sum(-1, keepdim=True)
    assert idx.dtype == torch.int64 and torch.equal(idx, ref_i)
    assert scores.dtype == dtype
    assert relerr(scores, ref_s.to(dtype)) <= (1e-5 if dtype is torch.float32 else 1e-2)
    assert torch.equal(counts.long(), torch.bincount(ref_i.reshape(-1), minlength=E))


def test_fused_router_declared_tie_rule(native):
    """Equal logits: the lowest expert index is taken first (torch.topk's choice here is unspecified, which is why the
    fused router is opt-in); NaN is never selected."""
    logits = torch.zeros(4, 16, device="cuda")
    logits[1, 9] = 1.0
    logits[2, :] = float("nan")
    logits[2, 5] = -3.0
    logits[3, 2] = float("nan")
    _, idx, _ = native.router_topk(logits, 3, False, False)
    assert idx[0].tolist() == [0, 1, 2]
    assert idx[1].tolist() == [9, 0, 1]
    assert idx[2].tolist()[0] == 5
    assert idx[3].tolist() == [0, 1, 3]


def test_layer_with_the_fused_router_matches_the_default_router(native):
    """Whole layer, forward and backward, with ``fused_router=True`` against the default (torch-op) router on logits
    that are tie-free after the bf16 GEMM's rounding is accounted for: the selected sets are equal, so outputs and
    gradients agree to the tolerance (the slot order inside a token differs, which only permutes summands)."""
    from moe_explore.functional.topk_moe import topk_moe_forward
    from moe_explore.params import MLPParams, MOEParams, TopkRouterParams

    T, d, E, k, I = 700, 256, 16, 4, 128
    g = torch.Generator(device="cuda").manual_seed(8)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g, device="cuda") * std).bfloat16()
    x, wr, w1, w2, grad = mk(T, d), mk(d, E, std=0.3), mk(E, d, 2 * I, std=0.05), mk(E, I, d, std=0.05), mk(T, d)
    logits = x @ wr
    top5 = torch.topk(logits.float(), k + 1, dim=-1).values
    keep = (top5[:, :-1] - top5[:, 1:]).min(-1).values > 0      # rows whose top-(k+1) logits are all distinct
    x, grad = x[keep].contiguous(), grad[keep].contiguous()
    results = []
    for fused in (False, True):
        leaves = [t.detach().clone().requires_grad_() for t in (x, wr, w1, w2)]
        params = MOEParams(TopkRouterParams(leaves[1], k, False, False), MLPParams(leaves[2], leaves[3], "swiglu"), E, k)
        out = topk_moe_forward(leaves[0], params, fused_router=fused)
        out.backward(grad)
        results.append([out.detach()] + [t.grad for t in leaves])
    for name, a, b in zip(("out", "dx", "d_router", "dw1", "dw2"), results[1], results[0]):
        assert relerr(a, b) <= TOL, name


@pytest.mark.parametrize("num_shared,act", [(1, "swiglu"), (2, "swiglu"), (3, "silu")])
def test_shared_expert_branch(num_shared, act, native):
    """topk_moe_forward with ``shared_expert_params`` (functional/topk_moe.py:56-62): the routed output plus the sum
    over the shared experts of act(x @ up) @ down, forward and backward, against fp32 torch on the same inputs."""
    from moe_explore.functional.topk_moe import topk_moe_forward
    from moe_explore.params import MLPParams, MOEParams, SharedExpertParams, TopkRouterParams

    T, d, E, k, I, Is = 400, 256, 8, 2, 128, 192
    g = torch.Generator(device="cuda").manual_seed(num_shared)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g, device="cuda") * std).bfloat16()
    x, wr, w1, w2, grad = mk(T, d), mk(d, E, std=0.1), mk(E, d, 2 * I, std=0.05), mk(E, I, d, std=0.05), mk(T, d)
    up = mk(num_shared, d, 2 * Is if "glu" in act else Is, std=0.05)
    down = mk(num_shared, Is, d, std=0.05)
    leaves = [t.detach().clone().requires_grad_() for t in (x, w1, w2, up, down)]
    params = MOEParams(TopkRouterParams(wr, k, False, False), MLPParams(leaves[1], leaves[2], "swiglu"), E, k,
                       SharedExpertParams(leaves[3], leaves[4], act))
    out = topk_moe_forward(leaves[0], params)
    out.backward(grad)
    # oracle: routed part by the oracle's expert loop (scores re-derived in fp32 from the same selection, so that the
    # input gradient includes the path through the router), shared part as the reference writes it
    from moe_explore.router import router

    with torch.no_grad():
        _, idx = router(x, params.router_params)
    f = [t.detach().float().requires_grad_() for t in (x, w1, w2, up, down)]
    scores = torch.softmax(torch.gather(f[0] @ wr.float(), -1, idx), -1)
    ref = O.expert_compute(f[0], scores, idx, f[1], f[2], "swiglu")
    h = O.activation(f[0] @ f[3], act) @ f[4]
    ref = ref + h.sum(0)
    ref.backward(grad.float())
    assert relerr(out, ref) <= TOL
    for name, a, b in zip(("dx", "dw1", "dw2", "d_up", "d_down"), [t.grad for t in leaves], [t.grad for t in f]):
        assert relerr(a, b) <= TOL, name


def test_expert_input_and_output_permute(native):
    """expert_input_permute / expert_output_permute (expert_permute.py:43-68): rows gathered into expert order are
    exact copies, the group prefix is the reference's, and permuting back with the router weights folds the k slots."""
    from moe_explore.expert_permute import expert_input_permute, expert_output_permute

    T, d, E, k = 777, 264, 16, 4
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(T, d, generator=g, device="cuda").bfloat16()
    top, idx = torch.topk(torch.randn(T, E, generator=g, device="cuda"), k, dim=-1, sorted=False)
    scores = torch.softmax(top, -1).bfloat16()
    grouped = expert_input_permute(x, idx, E, k)
    ref = O.get_token_indices(idx.cpu(), k, E, zero_prefix=True)
    assert torch.equal(grouped.group_indices.cpu(), ref.group_indices)
    assert torch.equal(grouped.indices.cpu(), ref.indices)
    assert torch.equal(grouped.tokens, x[(ref.indices // k).cuda()])
    back = expert_output_permute(grouped, scores, k, x.shape)
    # every token's k copies of its own row, weighted: x[t] * sum_s scores[t, s] (fp32 fold, one rounding)
    expect = (x.float() * scores.float().sum(-1, keepdim=True))
    assert back.shape == x.shape and relerr(back, expect) <= 1e-2

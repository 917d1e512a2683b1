"""This library's grouped GEMM against outputs of the REFERENCE's own Triton kernels on a B200, at the full
benchmark shapes (fixtures: tests/golden/ref_gpu_gemm_*.npz, made by tests/golden/make_gpu_golden.py).

Both implementations accumulate a row's products in fp32 in the same K order and round once to bf16, so the
comparison is on bit patterns."""
import os
import sys

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
from gpu_cases import CASES, make_case, sample  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(CASES))
def test_grouped_gemm_equals_reference_triton_output(name):
    from moe_explore.expert_permute import get_token_indices
    from moe_explore.triton_kernels.m_grouped_gemm import MGroupedGEMMParams, m_grouped_gemm

    path = os.path.join(GOLDEN, f"ref_gpu_gemm_{name}.npz")
    gold = np.load(path)
    device = torch.device("cuda", 0)
    c = make_case(name, device)
    drift = np.array([float(c["x"].double().sum()), float(c["w1"][0].double().sum()), float(c["h"].double().sum())])
    if not np.array_equal(drift, gold["checksum"]):
        pytest.skip("the seeded generator draws different inputs on this torch / GPU than where the fixture was made")
    with torch.no_grad():
        p = get_token_indices(c["idx"], c["k"], c["E"], zero_prefix=True)
        assert np.array_equal(p.group_indices.cpu().numpy(), gold["group_indices"])
        gathered = m_grouped_gemm(c["x"], MGroupedGEMMParams(
            c["w1"], p.group_indices, p.indices, gather=True, scatter=False, num_tokens=c["T"], topk=c["k"],
            scales=None, activation=None))
        h_sorted = c["h"][p.indices].contiguous()
        scattered = m_grouped_gemm(h_sorted, MGroupedGEMMParams(
            c["w2"], p.group_indices, p.indices, gather=False, scatter=True, num_tokens=c["T"], topk=c["k"],
            scales=c["scores"], activation=None))
        g, s = sample(gathered, p.indices, scattered)
    assert g.shape == gold["gather"].shape and s.shape == gold["scatter"].shape
    assert np.array_equal(g, gold["gather"]), "gather GEMM differs from the reference kernel's output"
    assert np.array_equal(s, gold["scatter"]), "scatter GEMM differs from the reference kernel's output"

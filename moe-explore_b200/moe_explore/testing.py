"""Harness helpers: synthetic routings, weight initialisers, parameter builders and the tolerance rule.

Same names and call signatures as the reference's helpers (src/moe_explore/testing.py:87-357), so that its
benchmarks and tests can be pointed at this package; the implementations are this repository's own.  One
difference: the reference's ``random_olmoe_routing`` samples experts from a table of 64 popularities measured on a
trained OLMoE layer, which is not reproduced here -- ``popularity_routing`` takes the popularity vector as an
argument, and ``zipf_popularity`` builds the synthetic one the benchmarks of this repository use.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from moe_explore.params import ErnieRouterParams, GLUInterleavedParams, GLUParams, MLPParams, TopkRouterParams


# ---------------------------------------------------------------------------------------------------------
# routings: every function returns (topk_scores [T, k] in `dtype`, topk_indices [T, k] int64)
# ---------------------------------------------------------------------------------------------------------
def random_routing(num_tokens: int, num_experts: int, topk: int, device, dtype):
    """Top-k of softmaxed N(0,1) logits: a nearly balanced routing (testing.py:97-106)."""
    probs = F.softmax(torch.randn(num_tokens, num_experts, device=device, dtype=torch.float32), dim=-1)
    scores, indices = torch.topk(probs, k=topk, dim=-1, sorted=False)
    return scores.to(dtype), indices


def perfect_routing(num_tokens: int, num_experts: int, topk: int, device, dtype):
    """Round-robin: flat position j goes to expert j % E, so every expert gets the same number of rows -- the case a
    batched GEMM can be compared with (testing.py:87-95)."""
    assert (num_tokens * topk) % num_experts == 0, "rows must divide evenly over the experts"
    indices = (torch.arange(num_tokens * topk, device=device) % num_experts).view(num_tokens, topk)
    scores, _ = random_routing(num_tokens, num_experts, topk, device, dtype)
    return scores, indices


def popularity_routing(num_tokens: int, popularity: torch.Tensor, topk: int, device, dtype):
    """Every token draws ``topk`` distinct experts with probabilities proportional to ``popularity`` [E]."""
    weights = popularity.to(device=device, dtype=torch.float32).clamp_min(0).expand(num_tokens, -1)
    indices = torch.multinomial(weights, num_samples=topk, replacement=False)
    scores, _ = random_routing(num_tokens, popularity.numel(), topk, device, dtype)
    return scores, indices


def random_skewed_routing(num_tokens: int, num_experts: int, topk: int, num_skewed_experts: int, skew_factor: int,
                          device, dtype):
    """``num_skewed_experts`` randomly chosen experts are ``skew_factor`` times as likely as the others
    (testing.py:108-132)."""
    popularity = torch.ones(num_experts)
    popularity[torch.randperm(num_experts)[:num_skewed_experts]] = float(skew_factor)
    return popularity_routing(num_tokens, popularity, topk, device, dtype)


def zipf_popularity(num_experts: int, exponent: float, generator=None) -> torch.Tensor:
    """p_e proportional to rank^-exponent over a random permutation of the experts."""
    p = torch.arange(1, num_experts + 1, dtype=torch.float32) ** (-exponent)
    return (p / p.sum())[torch.randperm(num_experts, generator=generator)]


def random_groups(num_tokens: int, num_groups: int, device) -> torch.Tensor:
    """int32 [G+1] exclusive prefix [0, r_1 <= ... <= r_{G-1}, num_tokens] with distinct random interior cuts
    (testing.py:212-224)."""
    cuts = torch.sort(torch.randperm(num_tokens - 2, device=device)[: num_groups - 1] + 1).values
    groups = torch.empty(num_groups + 1, dtype=torch.int32, device=device)
    groups[0], groups[-1] = 0, num_tokens
    groups[1:-1] = cuts.to(torch.int32)
    return groups


# ---------------------------------------------------------------------------------------------------------
# weights and parameter bundles
# ---------------------------------------------------------------------------------------------------------
def uniform_weight_init(size, device, dtype):
    """Bounded values (kinder to tolerances than a normal draw): U(-0.02, 0.02) for vectors, Xavier-uniform over the
    last two dims otherwise (testing.py:226-256)."""
    weight = torch.empty(size, device=device, dtype=dtype)
    if len(size) == 1:
        return weight.uniform_(-0.02, 0.02)
    bound = math.sqrt(3.0) * math.sqrt(2.0 / (size[-2] + size[-1]))
    return weight.uniform_(-bound, bound)


def normal_weight_init(size, device, dtype):
    """N(0, 0.02) (testing.py:258-261)."""
    return torch.empty(size, device=device, dtype=dtype).normal_(mean=0.0, std=0.02)


def random_mlp(num_experts, hidden_dim, intermediate_dim, activation, device, dtype, dist=uniform_weight_init):
    """``MLPParams`` with weight1 [E, d, I] (or [E, d, 2I] for a gated activation) and weight2 [E, I, d]."""
    width = 2 * intermediate_dim if "glu" in str(activation) else intermediate_dim
    return MLPParams(dist((num_experts, hidden_dim, width), device=device, dtype=dtype),
                     dist((num_experts, intermediate_dim, hidden_dim), device=device, dtype=dtype), activation)


def random_glu(num_experts, hidden_dim, intermediate_dim, activation, device, dtype, dist=uniform_weight_init):
    return GLUParams(dist((num_experts, hidden_dim, intermediate_dim), device=device, dtype=dtype),
                     dist((num_experts, hidden_dim, intermediate_dim), device=device, dtype=dtype),
                     dist((num_experts, intermediate_dim, hidden_dim), device=device, dtype=dtype), activation)


def random_interleaved_glu(num_experts, hidden_dim, intermediate_dim, activation, device, dtype, dist=uniform_weight_init):
    return GLUInterleavedParams(dist((num_experts, hidden_dim, 2 * intermediate_dim), device=device, dtype=dtype),
                                dist((num_experts, intermediate_dim, hidden_dim), device=device, dtype=dtype), activation)


def random_topk_router(num_experts, hidden_dim, topk, softmax_before_topk, normalize_routing, device, dtype,
                       dist=uniform_weight_init):
    return TopkRouterParams(dist((hidden_dim, num_experts), device=device, dtype=dtype), topk, softmax_before_topk,
                            normalize_routing)


def random_ernie_router(num_experts, hidden_dim, topk, device, dtype, dist=uniform_weight_init):
    return ErnieRouterParams(dist((hidden_dim, num_experts), device=device, dtype=torch.float32),
                             dist((num_experts,), device=device, dtype=torch.float32), topk)


# ---------------------------------------------------------------------------------------------------------
# tolerance rule
# ---------------------------------------------------------------------------------------------------------
def tolerances(a: torch.Tensor, b: torch.Tensor):
    """(atol, rtol) of the reference's rule (testing.py:340-357): both grow with the dtype's epsilon and the row
    length, atol also with the largest value, capped at 1e-2."""
    eps = {torch.bfloat16: 0.0078125, torch.float16: 0.0009765625, torch.float32: 1e-6}.get(a.dtype)
    if eps is None:
        raise ValueError(f"Invalid dtype: {a.dtype}")
    k = a.size(-1)
    largest = max(float(a.max()), float(b.max()))
    return min(1e-2, k * largest * eps * 1e-2), math.sqrt(k) * eps * 1e-1


def assert_close(a: torch.Tensor, b: torch.Tensor) -> None:
    atol, rtol = tolerances(a, b)
    torch.testing.assert_close(a, b, atol=atol, rtol=rtol)

"""Parameter bundles of the MoE layer.

Field names and order follow the reference dataclasses (src/moe_explore/params.py:6-59) so
that code constructing them positionally keeps working.  ``MOEParams`` additionally accepts
an optional ``shared_expert_params`` (the reference reads that attribute in
functional/topk_moe.py:56 although its dataclass does not declare it).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from moe_explore.functional.activation import Activation


@dataclass
class FFNParams:
    """Base of the expert feed-forward parameter bundles."""


@dataclass
class MLPParams(FFNParams):
    """Two-matrix expert: ``weight1`` [E, d, I] (or [E, d, 2I] interleaved gate/up for *glu),
    ``weight2`` [E, I, d]."""
    weight1: torch.Tensor
    weight2: torch.Tensor
    activation: Activation


@dataclass
class GLUParams(FFNParams):
    """Gated expert with separate gate / up matrices [E, d, I] and down [E, I, d]."""
    gate_weight: torch.Tensor
    up_weight: torch.Tensor
    down_weight: torch.Tensor
    activation: Activation


@dataclass
class GLUInterleavedParams(FFNParams):
    """Gated expert with gate (even columns) and up (odd columns) interleaved in one [E, d, 2I] matrix."""
    interleaved_weight: torch.Tensor
    down_weight: torch.Tensor
    activation: Activation


@dataclass
class SharedExpertParams(FFNParams):
    """Shared expert(s) applied to every token: ``up_weight`` [S, d, I] (or [S, d, 2I] interleaved for *glu),
    ``down_weight`` [S, I, d].  The reference reads exactly these three attributes
    (functional/topk_moe.py:56-62) without declaring a type for them."""
    up_weight: torch.Tensor
    down_weight: torch.Tensor
    activation: Activation


@dataclass
class RouterParams:
    """Base of the router parameter bundles."""


@dataclass
class TopkRouterParams(RouterParams):
    router_weight: torch.Tensor  # [d, E]
    topk: int
    softmax_before_topk: bool = True
    normalize_routing: bool = False


@dataclass
class ErnieRouterParams(RouterParams):
    router_weight: torch.Tensor  # [d, E], fp32
    bias: torch.Tensor           # [E], fp32, added to the probabilities for selection only
    topk: int


@dataclass
class MOEParams:
    router_params: RouterParams
    expert_params: FFNParams
    num_experts: int
    topk: int
    shared_expert_params: Optional[FFNParams] = None


@dataclass
class ExpertMatmulParams:
    tokens: torch.Tensor
    weight: torch.Tensor
    group_indices: torch.Tensor
    token_to_group_indices: torch.Tensor
    scales: Optional[torch.Tensor]


def interleave_gate_up(gate_weight: torch.Tensor, up_weight: torch.Tensor) -> torch.Tensor:
    """[E, d, I] gate and up matrices -> one [E, d, 2I] matrix, gate in even columns, up in odd
    columns: the layout ``activation(x, "swiglu")`` expects (functional/activation.py:17-25)."""
    assert gate_weight.shape == up_weight.shape
    return torch.stack((gate_weight, up_weight), dim=-1).reshape(*gate_weight.shape[:-1], -1).contiguous()

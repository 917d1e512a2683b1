"""Activation names and their torch definitions.

Same enum values and GLU column convention as the reference
(src/moe_explore/functional/activation.py:5-26): for ``swiglu`` / ``geglu`` the EVEN columns
are the gate and the ODD columns the linear branch; the result has half the width.
This torch form is what the fused CUDA epilogues are checked against; it also serves callers
that need the activation on its own (e.g. a shared expert).
"""
from __future__ import annotations

from enum import StrEnum

import torch
import torch.nn.functional as F


class Activation(StrEnum):
    SILU = "silu"
    GELU = "gelu"
    SWIGLU = "swiglu"
    GEGLU = "geglu"


def is_glu(act) -> bool:
    return act is not None and "glu" in str(act)


def activation(x: torch.Tensor, activation: Activation) -> torch.Tensor:
    assert activation in list(Activation), f"Invalid activation: {activation}"
    act = Activation(activation)
    if act is Activation.SILU:
        return F.silu(x)
    if act is Activation.GELU:
        return F.gelu(x)
    assert x.shape[-1] % 2 == 0
    gate, linear = x[..., 0::2], x[..., 1::2]
    gate = F.silu(gate) if act is Activation.SWIGLU else F.gelu(gate)
    return gate * linear

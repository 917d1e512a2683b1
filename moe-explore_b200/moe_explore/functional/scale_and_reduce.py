"""Weighted fold of the top-k slots back into one row per token.

Reference: src/moe_explore/functional/scale_and_reduce.py:3-5 --
``(input.view(T, k, -1) * scales[..., None]).sum(1)``.  On CUDA 16-bit tensors this runs the
library's combine kernel (fp32 accumulation, one rounding); it is differentiable.
"""
from __future__ import annotations

import torch

from moe_explore import _native


class _ScaleAndReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, scales, num_tokens, topk):
        rows = torch.arange(num_tokens * topk, dtype=torch.int32, device=input.device)
        out = torch.empty(num_tokens, input.size(1), dtype=input.dtype, device=input.device)
        _native.combine_topk(input.contiguous(), scales.contiguous(), rows, out, topk)
        ctx.save_for_backward(input, scales)
        ctx.topk = topk
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input, scales = ctx.saved_tensors
        k = ctx.topk
        g = grad_out.float()
        d_input = (g[:, None, :] * scales.float()[..., None]).reshape(input.shape).to(input.dtype)
        d_scales = (g[:, None, :] * input.float().view(g.size(0), k, -1)).sum(-1).to(scales.dtype)
        return d_input, d_scales, None, None


def scale_and_reduce(input: torch.Tensor, scales: torch.Tensor, num_tokens: int, topk: int, n: int) -> torch.Tensor:
    """``input`` [num_tokens*topk, n] in (token, slot) order, ``scales`` [num_tokens, topk] -> [num_tokens, n]."""
    assert input.dim() == 2 and input.size(0) == num_tokens * topk and input.size(1) == n
    assert scales.shape == (num_tokens, topk)
    _native.require_cuda(input, scales)
    return _ScaleAndReduce.apply(input, scales.to(input.dtype), num_tokens, topk)

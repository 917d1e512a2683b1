"""Generate the golden fixtures in this directory by running the REFERENCE implementation.

Needs a checkout of arthurfeeney/moe-explore, given as the first argument or in the
MOE_EXPLORE_REFERENCE environment variable; it is only run where that checkout exists, and its
outputs (*.npz next to this file) are committed so that the tests need nothing but the fixtures.

The reference is imported unmodified.  Three shims make its torch path run on a CPU-only host:
  * TORCHDYNAMO_DISABLE=1: its ``@torch.compile`` decorators become no-ops;
  * ``moe_explore.gpu_utils.get_gpu_sm_count`` is replaced before the Triton module is imported
    (the original asserts that a CUDA device exists at import time);
  * ``torch.histc`` is wrapped so that the int64-input / int32-out call in
    expert_permute.py:28-29 (CUDA-only as written) is served by ``torch.bincount``.

Usage:  TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py <reference_root>
"""
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MOE_EXPLORE_REFERENCE", "")
if not os.path.isdir(os.path.join(REF_ROOT, "src", "moe_explore")):
    raise SystemExit("usage: make_golden.py <path to a moe-explore checkout>")
sys.path.insert(0, os.path.join(REF_ROOT, "src"))

import moe_explore.gpu_utils as _gpu_utils  # noqa: E402  (the reference package)

_gpu_utils.get_gpu_sm_count = lambda device=None: 148

_orig_histc = torch.histc


def _histc_int(input, bins=100, min=0, max=0, *, out=None):
    if not input.is_floating_point():
        counts = torch.bincount(input.reshape(-1) - int(min), minlength=bins)[:bins]
        if out is not None:
            out.copy_(counts.to(out.dtype))
            return out
        return counts
    return _orig_histc(input, bins=bins, min=min, max=max, out=out)


torch.histc = _histc_int

from moe_explore.expert_permute import get_token_indices  # noqa: E402
from moe_explore.functional.activation import activation  # noqa: E402
from moe_explore.functional.scale_and_reduce import scale_and_reduce  # noqa: E402
from moe_explore.functional.topk_moe import topk_moe_torch  # noqa: E402
from moe_explore.params import ErnieRouterParams, MLPParams, MOEParams, TopkRouterParams  # noqa: E402
from moe_explore.router import router  # noqa: E402

assert "reference" in sys.modules["moe_explore"].__file__ or REF_ROOT in sys.modules["moe_explore"].__file__


def layer_inputs(seed, T, d, E, I, glu, dtype=torch.float32):
    """Draw order: x, router weight [d,E], W1 [E,d,(2)I], W2 [E,I,d]; N(0,1) / N(0,0.02)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g).to(dtype)
    wr = (torch.randn(d, E, generator=g) * 0.02).to(dtype)
    w1 = (torch.randn(E, d, 2 * I if glu else I, generator=g) * 0.02).to(dtype)
    w2 = (torch.randn(E, I, d, generator=g) * 0.02).to(dtype)
    return x, wr, w1, w2


def checksum(*tensors):
    return np.array([float(t.double().sum()) for t in tensors] + [float(t.double().abs().sum()) for t in tensors])


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach()
            if v.dtype is torch.bfloat16:
                v = v.float()
            v = v.numpy()
        out[k] = np.asarray(v)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def layer_case(name, seed, T, d, E, k, I, act, softmax_before_topk, normalize, store_inputs):
    glu = "glu" in act
    x, wr, w1, w2 = layer_inputs(seed, T, d, E, I, glu)
    rp = TopkRouterParams(wr, k, softmax_before_topk=softmax_before_topk, normalize_routing=normalize)
    params = MOEParams(rp, MLPParams(w1, w2, act), E, k)
    scores, idx = router(x, rp)
    pz = get_token_indices(idx, k, E, zero_prefix=True)
    pn = get_token_indices(idx, k, E, zero_prefix=False)
    try:
        out = topk_moe_torch(x, params)
    except AttributeError as err:
        # functional/topk_moe.py:56 reads params.shared_expert_params, which the reference's
        # MOEParams dataclass (params.py:46-51) does not declare; give the instance the attribute.
        print("  (setting shared_expert_params=None on the reference MOEParams:", err, ")")
        params.shared_expert_params = None
        out = topk_moe_torch(x, params)
    arrays = dict(meta=np.array([seed, T, d, E, k, I, int(softmax_before_topk), int(normalize)]), act=np.array(act),
                  scores=scores, indices=idx, group_zero_prefix=pz.group_indices, group_inclusive=pn.group_indices,
                  ref_perm=pz.indices, out=out, input_checksum=checksum(x, wr, w1, w2))
    if store_inputs:
        arrays.update(x=x, router_weight=wr, weight1=w1, weight2=w2)
    save(name, **arrays)


def main():
    torch.manual_seed(0)
    # whole layer, small shapes with the inputs stored
    layer_case("layer_small_swiglu", 1, 64, 64, 8, 2, 64, "swiglu", False, False, True)
    layer_case("layer_small_geglu_norm", 2, 48, 32, 4, 2, 32, "geglu", True, True, True)
    layer_case("layer_small_silu", 3, 33, 32, 16, 4, 48, "silu", True, False, True)
    layer_case("layer_small_gelu", 4, 40, 32, 8, 8, 16, "gelu", False, False, True)
    # first configuration of the benchmark suite: T=512 d=256 E=8 top-2 I=512 fp32 seed 0; inputs are
    # re-drawn from the seed by the tests (a checksum guards against generator drift)
    layer_case("layer_c1", 0, 512, 256, 8, 2, 512, "swiglu", False, False, False)

    # routing metadata on ragged / empty / single-expert id patterns
    g = torch.Generator().manual_seed(7)
    cases = {
        "uniform": torch.randint(0, 8, (50, 2), generator=g),
        "empty_experts": torch.randint(0, 3, (37, 4), generator=g) * 5,       # only experts 0, 5, 10 of 16
        "one_expert": torch.full((21, 2), 3, dtype=torch.int64),
        "single_row": torch.tensor([[2]]),
        "many_experts": torch.randint(0, 256, (64, 8), generator=g),
    }
    num_experts = {"uniform": 8, "empty_experts": 16, "one_expert": 8, "single_row": 4, "many_experts": 256}
    arrays = {}
    for name, idx in cases.items():
        E, k = num_experts[name], idx.size(1)
        z = get_token_indices(idx, k, E, zero_prefix=True)
        n = get_token_indices(idx, k, E, zero_prefix=False)
        arrays[name + "_idx"] = idx
        arrays[name + "_E"] = np.array(E)
        arrays[name + "_group_zero_prefix"] = z.group_indices
        arrays[name + "_group_inclusive"] = n.group_indices
        arrays[name + "_ref_perm"] = z.indices
    save("token_indices", **arrays)

    # activations and scale_and_reduce
    x = torch.randn(12, 16, generator=g) * 2
    y = torch.randn(6 * 4, 10, generator=g)
    s = torch.rand(6, 4, generator=g)
    save("activations", x=x, silu=activation(x, "silu"), gelu=activation(x, "gelu"), swiglu=activation(x, "swiglu"),
         geglu=activation(x, "geglu"), y=y, s=s, scale_and_reduce=scale_and_reduce(y, s, 6, 4, 10))

    # routers
    xr = torch.randn(20, 24, generator=g)
    wr = torch.randn(24, 12, generator=g) * 0.3
    bias = torch.randn(12, generator=g) * 0.1
    arrays = dict(x=xr, router_weight=wr, bias=bias)
    for sb in (False, True):
        for nm in (False, True):
            sc, ix = router(xr, TopkRouterParams(wr, 3, softmax_before_topk=sb, normalize_routing=nm))
            arrays[f"topk_sb{int(sb)}_nm{int(nm)}_scores"] = sc
            arrays[f"topk_sb{int(sb)}_nm{int(nm)}_indices"] = ix
    sc, ix = router(xr, ErnieRouterParams(wr, bias, 3))
    arrays["ernie_scores"], arrays["ernie_indices"] = sc, ix
    save("routers", **arrays)


if __name__ == "__main__":
    main()

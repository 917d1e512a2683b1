"""Generate ref_gpu_gemm_<case>.npz by running the REFERENCE's Triton grouped GEMM on a CUDA GPU.

Needs a checkout of arthurfeeney/moe-explore (first argument or MOE_EXPLORE_REFERENCE) and a GPU; the reference
is imported unmodified.  Only the kernel variants without an activation epilogue are run: with the Triton
release installed where these fixtures were made (3.6; the reference pins 3.4) the activation epilogue does not
compile (``accs[i] = EPILOGUE(accs[i])`` in triton_kernels/epilogue_split.py: tuple item assignment is rejected).
Per case: ``get_token_indices`` (expert_permute.py:19-41), ``m_grouped_gemm`` with gather=True on W1 and with
scatter=True on W2 (triton_kernels/m_grouped_gemm.py:332-393).

Usage:  python tests/golden/make_gpu_golden.py <reference_root> [case ...]
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MOE_EXPLORE_REFERENCE", "")
if not os.path.isdir(os.path.join(REF_ROOT, "src", "moe_explore")):
    raise SystemExit("usage: make_gpu_golden.py <path to a moe-explore checkout> [case ...]")
sys.path.insert(0, os.path.join(os.path.abspath(REF_ROOT), "src"))
sys.path.insert(0, HERE)

import moe_explore  # noqa: E402  (the reference package)

assert os.path.abspath(REF_ROOT) in os.path.abspath(moe_explore.__file__)
from gpu_cases import CASES, make_case, sample  # noqa: E402
from moe_explore.expert_permute import get_token_indices  # noqa: E402
from moe_explore.triton_kernels.m_grouped_gemm import MGroupedGEMMParams, m_grouped_gemm  # noqa: E402


def main():
    device = torch.device("cuda", 0)
    for name in (sys.argv[2:] or list(CASES)):
        c = make_case(name, device)
        with torch.no_grad():
            p = get_token_indices(c["idx"], c["k"], c["E"], zero_prefix=True)
            gathered = m_grouped_gemm(c["x"], MGroupedGEMMParams(
                c["w1"], p.group_indices, p.indices, gather=True, scatter=False, num_tokens=c["T"], topk=c["k"],
                scales=None, activation=None))
            h_sorted = c["h"][p.indices].contiguous()
            scattered = m_grouped_gemm(h_sorted, MGroupedGEMMParams(
                c["w2"], p.group_indices, p.indices, gather=False, scatter=True, num_tokens=c["T"], topk=c["k"],
                scales=c["scores"], activation=None))
            g, s = sample(gathered, p.indices, scattered)
        path = os.path.join(HERE, f"ref_gpu_gemm_{name}.npz")
        np.savez_compressed(path, gather=g, scatter=s, group_indices=p.group_indices.cpu().numpy(),
                            checksum=np.array([float(c["x"].double().sum()), float(c["w1"][0].double().sum()),
                                               float(c["h"].double().sum())]))
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")
        del c, gathered, scattered, h_sorted
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()

"""moe_explore -- the top-k MoE expert-compute path of arthurfeeney/moe-explore on B200 (sm_100a).

Module paths mirror the reference package (src/moe_explore/): ``params``, ``router``,
``expert_permute``, ``functional.{activation,scale_and_reduce,topk_moe}`` and
``triton_kernels.m_grouped_gemm`` (the name is kept for drop-in imports; nothing here uses
Triton).  All compute goes through libmoe_sm100.so (``_native``); there is no CPU path.
"""

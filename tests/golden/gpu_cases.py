"""Seeded inputs and the row/column sample shared by make_gpu_golden.py (which runs the reference's Triton
grouped GEMM on a GPU) and tests/test_reference_gpu_golden.py (which runs this library on the same inputs).

Imports neither implementation, so that either can be on sys.path under the name ``moe_explore``."""
import torch

# T tokens, d hidden, E experts, top-k, I intermediate: the benchmark shapes of the Mixtral, Qwen1.5-MoE and
# OLMoE layers (bf16)
CASES = {
    "mixtral_8x7b": dict(T=8192, d=4096, E=8, k=2, I=14336),
    "qwen15_moe_a27b": dict(T=16384, d=2048, E=60, k=4, I=1408),
    "olmoe_8192": dict(T=8192, d=2048, E=64, k=8, I=1024),
}
ROW_STEP, ROWS_KEPT, COLS_KEPT = 257, 64, 512


def make_case(name, device, dtype=torch.bfloat16):
    """x [T,d] ~ N(0,1); W1 [E,d,2I], W2 [E,I,d] ~ N(0,0.02) drawn per expert; N(0,1) router logits -> top-k
    indices and softmax scores; h [T*k, I] ~ N(0,1), the down GEMM's input in (token, slot) order."""
    c = CASES[name]
    T, d, E, k, I = c["T"], c["d"], c["E"], c["k"], c["I"]
    gen = torch.Generator(device=device).manual_seed(2024)
    x = torch.randn(T, d, generator=gen, device=device).to(dtype)
    w1 = torch.empty(E, d, 2 * I, dtype=dtype, device=device)
    w2 = torch.empty(E, I, d, dtype=dtype, device=device)
    for e in range(E):
        w1[e] = (torch.randn(d, 2 * I, generator=gen, device=device) * 0.02).to(dtype)
        w2[e] = (torch.randn(I, d, generator=gen, device=device) * 0.02).to(dtype)
    logits = torch.randn(T, E, generator=gen, device=device)
    top, idx = torch.topk(logits, k, dim=-1, sorted=False)
    scores = torch.softmax(top, dim=-1, dtype=torch.float32).to(dtype)
    h = torch.randn(T * k, I, generator=gen, device=device).to(dtype)
    return dict(x=x, w1=w1, w2=w2, idx=idx, scores=scores, h=h, **c)


def sample(gathered_sorted, perm, scattered):
    """gathered_sorted: output of the gather GEMM, rows in expert-sorted order (row r belongs to flat position
    perm[r]); scattered: output of the scatter GEMM, rows in flat (token, slot) order.  Returns the bf16 bit
    patterns (int16) of a fixed sample of both, with the gather rows put back into flat order first -- the order
    inside an expert's segment is implementation-defined, flat order is not."""
    flat = torch.empty_like(gathered_sorted)
    flat[perm] = gathered_sorted
    rows = torch.arange(0, flat.size(0), ROW_STEP, device=flat.device)[:ROWS_KEPT]
    gs = flat[rows][:, ::7][:, :COLS_KEPT].contiguous()
    step = max(scattered.size(1) // COLS_KEPT, 1)
    ss = scattered[rows][:, ::step][:, :COLS_KEPT].contiguous()
    return gs.view(torch.int16).cpu().numpy(), ss.view(torch.int16).cpu().numpy()

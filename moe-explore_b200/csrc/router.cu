// Fused router tail: logits -> (fp32 softmax) -> top-k -> (softmax over the k) -> (renormalise) -> scores, indices
// and the per-expert load histogram, one warp per token, one launch.
//
// Replaces the chain of torch launches behind topk_router (reference: src/moe_explore/router.py:17-35: softmax,
// torch.topk, softmax, division, cast).  The logits themselves (input @ router_weight) stay a library GEMM.
//
// OPT-IN.  The reference's routing is defined by torch.topk, whose choice among equal logits and whose output order
// (sorted=False) are implementation details of torch; the default router of this package therefore keeps the torch
// ops, which makes its indices bit-identical to the reference's on the same device.  This kernel declares its own
// rule instead:
//   * among equal values the LOWEST expert index is selected first;
//   * the k selected experts are returned in descending order of value (ties: ascending index);
//   * NaN logits are never selected.
// On inputs without ties among the selected values the SET of indices per token equals torch.topk's.
// Arithmetic is fp32 on the upcast logits; HBM-bound: T*E logits read once, 10*T*k bytes written.
#include "common.cuh"

#include <math_constants.h>

namespace moe {

constexpr int kRouterWarps = 8;
constexpr int kRouterMaxPerLane = 32;  // E <= 1024

template <typename T> __device__ __forceinline__ float load_logit(const T* p) { return Elem<T>::to_float(*p); }
template <> __device__ __forceinline__ float load_logit<float>(const float* p) { return *p; }
template <typename T> __device__ __forceinline__ void store_score(T* p, float v) { *p = Elem<T>::from_float(v); }
template <> __device__ __forceinline__ void store_score<float>(float* p, float v) { *p = v; }

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const T* __restrict__ logits, T* __restrict__ scores, int64_t* __restrict__ indices,
                   int32_t* __restrict__ expert_counts, int64_t num_tokens, int E, int topk, int softmax_before,
                   int normalize) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kRouterWarps + warp;
  if (t >= num_tokens) return;
  // expert e = i * 32 + lane lives in v[i]
  float v[PER_LANE];
  const T* row = logits + t * E;
  float vmax = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    float x = e < E ? load_logit<T>(row + e) : -CUDART_INF_F;
    if (x != x) x = -CUDART_INF_F;  // NaN: never selected
    v[i] = x;
    vmax = fmaxf(vmax, x);
  }
  float denom = 1.0f;
  if (softmax_before) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xFFFFFFFFu, vmax, off));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < E && v[i] > -CUDART_INF_F) sum += expf(v[i] - vmax);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    denom = sum;
  }
  // k rounds of warp arg-max; the winner's slot is cleared.  Lane s keeps the s-th winner (k <= 32).
  float my_val = 0.0f;
  int my_idx = 0;
  for (int s = 0; s < topk; ++s) {
    float best = -CUDART_INF_F;
    int best_e = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < E && v[i] > best) {  // strict: the lowest index of equal values within a lane stays
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, off);
      const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if (best_e == 0x7FFFFFFF) best_e = s < E ? s : 0;  // fewer than k finite logits: deterministic filler
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) v[i] = -CUDART_INF_F;
    }
    if (lane == s) {
      my_val = best;
      my_idx = best_e;
    }
  }
  // scores of the selected experts
  float score = 0.0f;
  const bool mine = lane < topk;
  if (softmax_before) {
    score = mine && my_val > -CUDART_INF_F ? expf(my_val - vmax) / denom : 0.0f;
  } else {
    float m = mine ? my_val : -CUDART_INF_F;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    float ex = mine && my_val > -CUDART_INF_F ? expf(my_val - m) : 0.0f;
    float sum = ex;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    score = sum > 0.0f ? ex / sum : 0.0f;
  }
  if (normalize) {
    float sum = mine ? score : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    score = score / sum;
  }
  if (mine) {
    store_score<T>(scores + t * topk + lane, score);
    indices[t * topk + lane] = my_idx;
    if (expert_counts != nullptr) atomicAdd(expert_counts + my_idx, 1);
  }
}

template <typename T>
static int launch_router(const void* logits, void* scores, int64_t* indices, int32_t* counts, int64_t T_, int E, int topk,
                         int softmax_before, int normalize, cudaStream_t s) {
  const int blocks = static_cast<int>((T_ + kRouterWarps - 1) / kRouterWarps);
  const T* l = static_cast<const T*>(logits);
  T* sc = static_cast<T*>(scores);
#define MOE_ROUTER(PL)                                                                                                   \
  router_topk_kernel<T, PL><<<blocks, kRouterWarps * 32, 0, s>>>(l, sc, indices, counts, T_, E, topk, softmax_before, normalize)
  if (E <= 64) MOE_ROUTER(2);
  else if (E <= 128) MOE_ROUTER(4);
  else if (E <= 256) MOE_ROUTER(8);
  else if (E <= 512) MOE_ROUTER(16);
  else MOE_ROUTER(32);
#undef MOE_ROUTER
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

}  // namespace moe

using namespace moe;

extern "C" int moe_router_topk(const void* logits, void* scores, int64_t* indices, int32_t* expert_counts,
                               int64_t num_tokens, int num_experts, int topk, int softmax_before_topk, int normalize,
                               int dtype, void* stream) {
  MOE_CHECK_ARG(num_tokens >= 0 && num_experts > 0 && topk > 0, "moe_router_topk: bad sizes T=%lld E=%d k=%d",
                (long long)num_tokens, num_experts, topk);
  if (num_experts > 32 * kRouterMaxPerLane || topk > 32 || topk > num_experts) {
    set_error("moe_router_topk: supports E <= %d and k <= min(32, E); got E=%d k=%d", 32 * kRouterMaxPerLane, num_experts, topk);
    return MOE_ERR_UNSUPPORTED;
  }
  if (num_tokens == 0) return MOE_OK;
  MOE_CHECK_ARG(logits && scores && indices, "moe_router_topk: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (expert_counts != nullptr) MOE_CUDA(cudaMemsetAsync(expert_counts, 0, sizeof(int32_t) * num_experts, s));
  if (dtype == MOE_DTYPE_BF16)
    return launch_router<__nv_bfloat16>(logits, scores, indices, expert_counts, num_tokens, num_experts, topk,
                                        softmax_before_topk, normalize, s);
  if (dtype == MOE_DTYPE_F16)
    return launch_router<__half>(logits, scores, indices, expert_counts, num_tokens, num_experts, topk, softmax_before_topk,
                                 normalize, s);
  if (dtype == MOE_DTYPE_F32)
    return launch_router<float>(logits, scores, indices, expert_counts, num_tokens, num_experts, topk, softmax_before_topk,
                                normalize, s);
  set_error("moe_router_topk: unknown dtype %d", dtype);
  return MOE_ERR_INVALID;
}

// Row movement around the grouped GEMMs: gather token rows into the padded expert-sorted
// layout, fold the top-k slots back into token order with the router weights, and the
// backward of that fold.  All kernels are HBM-bound: 16-byte vector accesses, one warp per
// row segment, fp32 accumulation where values are summed.
//
// Replace row_gather / row_scatter (reference: src/moe_explore/triton_kernels/row_gather_scatter.py:36-116)
// and scale_and_reduce (src/moe_explore/functional/scale_and_reduce.py:3-5).
#include "common.cuh"

namespace moe {

constexpr int kRowThreads = 256;

// dst[p, :] = src[row_src[p] / div, :], zeros for padding rows.  One CTA per padded row.
__global__ void __launch_bounds__(kRowThreads)
gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ row_src,
                   const int32_t* __restrict__ num_mtiles, uint4* __restrict__ dst, int vec_per_row, int div) {
  const int64_t rows_in_use = static_cast<int64_t>(*num_mtiles) * MOE_TILE_M;
  for (int64_t p = blockIdx.x; p < rows_in_use; p += gridDim.x) {
    const int32_t j = row_src[p];
    uint4* d = dst + p * vec_per_row;
    if (j < 0) {
      for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) d[v] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* s = src + static_cast<int64_t>(j / div) * vec_per_row;
      for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) d[v] = s[v];
    }
  }
}

// Token-major form of the same movement for the layer's own dispatch: dst[dst_row[t*topk + s], :] = src[t, :].
// Every token row is read from HBM once and written topk times (the row-major gather re-reads it topk
// times, and the tokens of an expert are scattered over the whole input).  The second part of the grid
// zeroes the padding rows.
__global__ void __launch_bounds__(kRowThreads)
dispatch_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ dst_row,
                     const int32_t* __restrict__ row_src, const int32_t* __restrict__ num_mtiles,
                     uint4* __restrict__ dst, int64_t num_tokens, int topk, int vec_per_row, int token_blocks) {
  if (static_cast<int>(blockIdx.x) < token_blocks) {
    for (int64_t t = blockIdx.x; t < num_tokens; t += token_blocks) {
      const uint4* s = src + t * vec_per_row;
      const int32_t* rows = dst_row + t * topk;
      for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) {
        const uint4 u = s[v];
        for (int k = 0; k < topk; ++k) {
          const int32_t p = rows[k];  // negative: the routing metadata dropped this (token, slot)
          if (p >= 0) dst[static_cast<int64_t>(p) * vec_per_row + v] = u;
        }
      }
    }
  } else {
    // padding rows: one warp per row, only rows whose row_src is negative
    const int64_t rows_in_use = static_cast<int64_t>(*num_mtiles) * MOE_TILE_M;
    const int warps = (gridDim.x - token_blocks) * (kRowThreads / 32);
    const int warp = (blockIdx.x - token_blocks) * (kRowThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    for (int64_t p = warp; p < rows_in_use; p += warps) {
      if (row_src[p] >= 0) continue;
      uint4* d = dst + p * vec_per_row;
      for (int v = lane; v < vec_per_row; v += 32) d[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Row window of a pull: everything, or the rows of the experts of chunk `chunk_index` of `chunk_count` (the same
// slicing the grouped GEMMs use, so a caller can pipeline the pull of chunk c+1 against the GEMMs of chunk c).
// False when the metadata was built for another padded row count.
// chunk_count < 0 encodes an explicit expert range: experts [chunk_index, -chunk_count).  pair_end > pair_begin selects
// the rows of the row-tile pairs [pair_begin, pair_end) of the pair list instead (a slice that may cut through an expert).
struct RowWindow {
  int chunk_index, chunk_count;
  int pair_begin, pair_end;
};
__device__ __forceinline__ bool peer_row_window(const int32_t* __restrict__ num_mtiles, const int32_t* __restrict__ tile_pairs,
                                                int num_experts, int mtiles_bound, const RowWindow& w,
                                                int64_t& row_begin, int64_t& row_end) {
  const int chunk_index = w.chunk_index, chunk_count = w.chunk_count;
  const bool by_pairs = w.pair_end > w.pair_begin;
  row_begin = 0;
  row_end = static_cast<int64_t>(num_mtiles[0]) * MOE_TILE_M;
  if (chunk_count > 1 || chunk_count < 0 || by_pairs) {
    if (num_mtiles[2] != mtiles_bound) return false;
    const int32_t* pair_prefix = tile_pairs + mtiles_bound;
    const int pairs = num_mtiles[1];
    int p0, p1;
    if (by_pairs) {
      p0 = w.pair_begin < pairs ? w.pair_begin : pairs;
      p1 = w.pair_end < pairs ? w.pair_end : pairs;
    } else {
      int e0, e1;
      if (chunk_count < 0) {
        e0 = chunk_index;
        e1 = -chunk_count < num_experts ? -chunk_count : num_experts;
      } else {
        e0 = static_cast<int>(static_cast<long long>(num_experts) * chunk_index / chunk_count);
        e1 = static_cast<int>(static_cast<long long>(num_experts) * (chunk_index + 1) / chunk_count);
      }
      p0 = pair_prefix[e0];
      p1 = pair_prefix[e1];
    }
    if (p1 < pairs) row_end = static_cast<int64_t>(tile_pairs[p1] & 0xFFFFF) * MOE_TILE_M;
    row_begin = p0 < pairs ? static_cast<int64_t>(tile_pairs[p0] & 0xFFFFF) * MOE_TILE_M : row_end;
  }
  return true;
}

// dst[p, :] = scale[p] * bases[src_rank[p]][src_row[p], :], zeros where src_rank[p] < 0.  `bases` holds
// one base pointer per rank of the node: the source rows live in peers' memory and are read with
// ordinary 16-byte loads over NVLink (this GPU's own rows through the same path).
// 128-thread CTAs of at most 64 registers: one of them still fits beside a grouped-GEMM CTA (320 threads x ~165
// registers), so the pull also makes progress on the SMs it does not have to itself, and on a free SM eight fit.
// The grid has more CTAs than can be resident; those that wait take over from the ones that finish, which hands
// most rows to the SMs where the kernel runs fast.
//
// THREADS = 1024 is the DEDICATED form: one CTA takes the whole register file of an SM, so it neither fits beside
// a GEMM CTA nor lets one start next to it; launched with as many CTAs as the GEMMs leave SMs free, the pull then
// has those SMs to itself (131 KB of loads in flight on each) and the GEMMs are not slowed by pull CTAs that share
// their SMs' L2 ingress and issue slots.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS == 128 ? 8 : 1)
gather_rows_peer_kernel(const uint4* const* __restrict__ bases, const int32_t* __restrict__ src_rank,
                        const int32_t* __restrict__ src_row, const float* __restrict__ scale,
                        const int32_t* __restrict__ num_mtiles, const int32_t* __restrict__ tile_pairs,
                        int num_experts, int mtiles_bound, RowWindow window, uint4* __restrict__ dst,
                        int vec_per_row) {
  int64_t row_begin, row_end;
  if (!peer_row_window(num_mtiles, tile_pairs, num_experts, mtiles_bound, window, row_begin, row_end)) return;
  // Two rows per iteration, up to four 16-byte loads per thread and row, ALL issued before the first store: a
  // remote load takes microseconds, so what a thread keeps in flight is what the pull is worth (with one row of
  // 7168 elements a thread had only 3.5 loads to issue; load -> store -> load in program order gave it one).
  constexpr int kRows = 2, kLoads = 4;
  for (int64_t p0 = row_begin + blockIdx.x; p0 < row_end; p0 += static_cast<int64_t>(gridDim.x) * kRows) {
    for (int v0 = threadIdx.x; v0 < vec_per_row; v0 += kLoads * THREADS) {
      uint4 u[kRows][kLoads];
      float f[kRows];
      bool live[kRows];
#pragma unroll
      for (int q = 0; q < kRows; ++q) {
        const int64_t p = p0 + static_cast<int64_t>(q) * gridDim.x;
        const int32_t r = p < row_end ? src_rank[p] : -1;
        live[q] = r >= 0;
        f[q] = (live[q] && scale != nullptr) ? scale[p] : 1.0f;
        const uint4* s = live[q] ? bases[r] + static_cast<int64_t>(src_row[p]) * vec_per_row : nullptr;
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
          const int v = v0 + i * THREADS;
          u[q][i] = (live[q] && v < vec_per_row) ? s[v] : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int q = 0; q < kRows; ++q) {
        const int64_t p = p0 + static_cast<int64_t>(q) * gridDim.x;
        if (p >= row_end) continue;
        uint4* d = dst + p * vec_per_row;
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
          const int v = v0 + i * THREADS;
          if (v >= vec_per_row) continue;
          if (live[q] && scale != nullptr) {
            const uint32_t w[4] = {u[q][i].x, u[q][i].y, u[q][i].z, u[q][i].w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 x = Elem<T>::unpack2(w[k]);
              o[k] = Elem<T>::pack2(f[q] * x.x, f[q] * x.y);
            }
            u[q][i] = make_uint4(o[0], o[1], o[2], o[3]);
          }
          d[v] = u[q][i];  // padding rows (src_rank < 0) are written as zeros
        }
      }
    }
  }
}

// The same pull with the copy engine of the SM doing the moving: every warp owns one shared-memory slot of one
// row; one lane fetches the row with a bulk asynchronous copy (global -> shared, completion on an mbarrier), the
// warp scales it in place when asked to, and one lane sends it on with a bulk copy shared -> global.  A row of
// 14 KB is in flight per warp without a register holding any of it, so a CTA keeps ~170 KB of remote reads
// outstanding -- what a pull over NVLink (microseconds of latency) needs when it has only a few SMs to itself.
// Launched with at most as many CTAs as there are SMs free for it (one CTA per SM: the slots take the shared memory).
constexpr int kBulkMaxWarps = 16;
template <typename T>
__global__ void __launch_bounds__(kBulkMaxWarps * 32)
pull_rows_bulk_kernel(const uint4* const* __restrict__ bases, const int32_t* __restrict__ src_rank,
                      const int32_t* __restrict__ src_row, const float* __restrict__ scale,
                      const int32_t* __restrict__ num_mtiles, const int32_t* __restrict__ tile_pairs, int num_experts,
                      int mtiles_bound, RowWindow window, uint4* __restrict__ dst, int vec_per_row,
                      long long wait_limit, int32_t* status) {
  extern __shared__ __align__(128) uint8_t slots_raw[];
  __shared__ __align__(8) uint64_t bars[kBulkMaxWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const uint32_t row_bytes = static_cast<uint32_t>(vec_per_row) * 16u;
  const uint32_t slot = smem_u32(slots_raw) + warp * row_bytes;
  uint4* slot_ptr = reinterpret_cast<uint4*>(slots_raw + static_cast<size_t>(warp) * row_bytes);
  const uint32_t bar = smem_u32(&bars[warp]);
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  int64_t row_begin, row_end;
  if (!peer_row_window(num_mtiles, tile_pairs, num_experts, mtiles_bound, window, row_begin, row_end)) return;
  uint32_t phase = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * warps;
  for (int64_t p = row_begin + static_cast<int64_t>(blockIdx.x) * warps + warp; p < row_end; p += stride) {
    const int32_t r = src_rank[p];
    uint4* d = dst + p * vec_per_row;
    if (r < 0) {
      for (int v = lane; v < vec_per_row; v += 32) d[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* src = bases[r] + static_cast<int64_t>(src_row[p]) * vec_per_row;
    if (lane == 0) {
      bulk_wait_read_all();  // the store of this warp's previous row has left the slot
      mbar_arrive_expect_tx(bar, row_bytes);
      asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(slot), "l"(src), "r"(row_bytes), "r"(bar)
                   : "memory");
    }
    __syncwarp();
    // bounded wait for the row
    bool arrived = mbar_try_wait(bar, phase);
    if (!arrived) {
      const long long t0 = clock64();
      while (!(arrived = mbar_try_wait(bar, phase))) {
        if (clock64() - t0 > wait_limit) break;
      }
    }
    if (!__all_sync(0xFFFFFFFFu, arrived)) {
      if (lane == 0 && status != nullptr) atomicCAS(status, 0, DS_TIMEOUT_PRODUCER);
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let the copy land before the CTA gives up its shared memory
      break;
    }
    phase ^= 1;
    if (scale != nullptr) {
      const float f = scale[p];
      for (int v = lane; v < vec_per_row; v += 32) {
        const uint4 u = slot_ptr[v];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = Elem<T>::unpack2(w[k]);
          o[k] = Elem<T>::pack2(f * x.x, f * x.y);
        }
        slot_ptr[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();
    }
    __syncwarp();
    if (lane == 0) {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d), "r"(slot), "r"(row_bytes) : "memory");
      bulk_commit();
    }
  }
  if (lane == 0) bulk_wait_all();
}

// out[j, :] = src[dst_row[j], :]
__global__ void __launch_bounds__(kRowThreads)
unpad_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ dst_row, uint4* __restrict__ out,
                  int64_t num_rows, int vec_per_row) {
  for (int64_t j = blockIdx.x; j < num_rows; j += gridDim.x) {
    const int32_t p = dst_row[j];
    uint4* d = out + j * vec_per_row;
    if (p < 0) {  // no source row (dropped by the routing metadata): zeros
      for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) d[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* s = src + static_cast<int64_t>(p) * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) d[v] = s[v];
  }
}

template <typename T>
__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& u, float scale) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = Elem<T>::unpack2(w[i]);
    acc[2 * i] = fmaf(scale, f.x, acc[2 * i]);
    acc[2 * i + 1] = fmaf(scale, f.y, acc[2 * i + 1]);
  }
}

// out[t, :] = sum_s scale(t, s) * ys[dst_row[t*topk + s], :]
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
combine_topk_kernel(const uint4* __restrict__ ys, const T* __restrict__ scores, const int32_t* __restrict__ dst_row,
                    uint4* __restrict__ out, int64_t num_tokens, int topk, int vec_per_row) {
  for (int64_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int s = 0; s < topk; ++s) {
        const int64_t j = t * topk + s;
        const int32_t p = dst_row[j];
        if (p < 0) continue;  // slot dropped by the routing metadata: contributes nothing
        const float scale = scores != nullptr ? Elem<T>::to_float(scores[j]) : 1.0f;
        const uint4 u = ys[static_cast<int64_t>(p) * vec_per_row + v];
        fma8<T>(acc, u, scale);
      }
      uint4 r;
      r.x = Elem<T>::pack2(acc[0], acc[1]);
      r.y = Elem<T>::pack2(acc[2], acc[3]);
      r.z = Elem<T>::pack2(acc[4], acc[5]);
      r.w = Elem<T>::pack2(acc[6], acc[7]);
      out[t * vec_per_row + v] = r;
    }
  }
}

// gs[p, :] = scores[j] * dout[t, :];  dscores[j] = dot(dout[t, :], ys[p, :]);  j = row_src[p], t = j / topk.
// One warp per padded row (8 rows per CTA): the dot product is a warp-shuffle reduction, no block barrier.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
combine_bwd_kernel(const uint4* __restrict__ dout, const T* __restrict__ scores, const uint4* __restrict__ ys,
                   const int32_t* __restrict__ row_src, const int32_t* __restrict__ num_mtiles,
                   uint4* __restrict__ gs, T* __restrict__ dscores, int topk, int vec_per_row) {
  constexpr int kWarps = kRowThreads / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows_in_use = static_cast<int64_t>(*num_mtiles) * MOE_TILE_M;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * kWarps + warp; p < rows_in_use;
       p += static_cast<int64_t>(gridDim.x) * kWarps) {
    const int32_t j = row_src[p];
    uint4* g = gs != nullptr ? gs + p * vec_per_row : nullptr;
    if (j < 0) {  // padding row (uniform across the warp)
      if (g != nullptr)
        for (int v = lane; v < vec_per_row; v += 32) g[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float scale = Elem<T>::to_float(scores[j]);
    const uint4* d = dout + static_cast<int64_t>(j / topk) * vec_per_row;
    const uint4* y = ys + p * vec_per_row;
    float dot = 0.0f;
    for (int v = lane; v < vec_per_row; v += 32) {
      const uint4 du = d[v];
      const uint4 yu = y[v];
      const uint32_t dw[4] = {du.x, du.y, du.z, du.w};
      const uint32_t yw[4] = {yu.x, yu.y, yu.z, yu.w};
      uint32_t ow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 df = Elem<T>::unpack2(dw[i]);
        const float2 yf = Elem<T>::unpack2(yw[i]);
        dot = fmaf(df.x, yf.x, dot);
        dot = fmaf(df.y, yf.y, dot);
        ow[i] = Elem<T>::pack2(scale * df.x, scale * df.y);
      }
      if (g != nullptr) g[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
    if (lane == 0) dscores[j] = Elem<T>::from_float(dot);
  }
}

// A few words from device memory into PINNED host memory, written by a kernel through the unified address space.
// For the one small host read a step needs (split sizes): a memcpy would be queued on a copy engine, behind
// whatever large host transfer another stream has in flight there (the next batch's upload, the last result's
// read-back), and the step would wait for all of it.
__global__ void store_words_to_host_kernel(const unsigned long long* __restrict__ src, unsigned long long* __restrict__ dst,
                                           int64_t words) {
  for (int64_t i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
  __threadfence_system();
}

// Zeroes the padding rows (row_src < 0) of a [rows, vec_per_row] buffer in the padded layout: one warp per row.
__global__ void __launch_bounds__(kRowThreads)
zero_padding_rows_kernel(const int32_t* __restrict__ row_src, const int32_t* __restrict__ num_mtiles, uint4* __restrict__ dst,
                         int vec_per_row) {
  const int64_t rows_in_use = static_cast<int64_t>(*num_mtiles) * MOE_TILE_M;
  const int warps = gridDim.x * (kRowThreads / 32);
  const int lane = threadIdx.x & 31;
  for (int64_t p = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); p < rows_in_use; p += warps) {
    if (row_src[p] >= 0) continue;
    uint4* d = dst + p * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) d[v] = make_uint4(0, 0, 0, 0);
  }
}

static int row_grid(int64_t rows) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace moe

using namespace moe;

#define MOE_ROW_COMMON_CHECKS(name, cols, dtype)                                                          \
  MOE_CHECK_ARG((cols) > 0, name ": cols=%d must be positive", (cols));                                  \
  if ((cols) % 8 != 0) {                                                                                 \
    set_error(name ": cols=%d must be a multiple of 8 (16-byte rows)", (cols));                          \
    return MOE_ERR_UNSUPPORTED;                                                                          \
  }                                                                                                      \
  MOE_CHECK_ARG((dtype) == MOE_DTYPE_BF16 || (dtype) == MOE_DTYPE_F16, name ": unknown dtype %d", (dtype))

extern "C" int moe_zero_padding_rows(const int32_t* row_src, const int32_t* num_mtiles, void* dst, int64_t padded_rows,
                                     int cols, int dtype, void* stream) {
  MOE_CHECK_ARG(row_src && num_mtiles && dst, "moe_zero_padding_rows: null pointer argument");
  MOE_CHECK_ARG(aligned16(dst) && padded_rows > 0, "moe_zero_padding_rows: dst must be 16-byte aligned, padded_rows positive");
  MOE_ROW_COMMON_CHECKS("moe_zero_padding_rows", cols, dtype);
  zero_padding_rows_kernel<<<sm_count() * 2, kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      row_src, num_mtiles, static_cast<uint4*>(dst), cols / 8);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_copy_blocks(void* const* dst, const void* const* src, const size_t* bytes, int count, void* stream) {
  MOE_CHECK_ARG(count >= 0 && (count == 0 || (dst && src && bytes)), "moe_copy_blocks: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < count; ++i) {
    if (bytes[i] == 0) continue;
    MOE_CHECK_ARG(dst[i] != nullptr && src[i] != nullptr, "moe_copy_blocks: block %d has a null address", i);
    // one plain asynchronous copy per block: the copy engines move it, no SM is involved
    MOE_CUDA(cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDeviceToDevice, s));
  }
  return MOE_OK;
}

extern "C" int moe_store_to_host(const void* src, void* dst_pinned_host, size_t bytes, void* stream) {
  MOE_CHECK_ARG(src != nullptr && dst_pinned_host != nullptr, "moe_store_to_host: null pointer argument");
  MOE_CHECK_ARG(bytes % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 7u) == 0 &&
                    (reinterpret_cast<uintptr_t>(dst_pinned_host) & 7u) == 0,
                "moe_store_to_host: size and pointers must be multiples of 8 bytes");
  if (bytes == 0) return MOE_OK;
  cudaPointerAttributes attr;
  MOE_CUDA(cudaPointerGetAttributes(&attr, dst_pinned_host));
  MOE_CHECK_ARG(attr.type == cudaMemoryTypeHost, "moe_store_to_host: the destination is not page-locked host memory");
  const int64_t words = static_cast<int64_t>(bytes / 8);
  const int blocks = static_cast<int>(words < 256 * 64 ? (words + 255) / 256 : 64);
  store_words_to_host_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(src), static_cast<unsigned long long*>(attr.devicePointer), words);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_gather_rows(const void* src, int64_t src_rows, const int32_t* row_src, const int32_t* num_mtiles,
                               void* dst, int64_t padded_rows, int cols, int div, int dtype, void* stream) {
  MOE_CHECK_ARG(src && row_src && num_mtiles && dst, "moe_gather_rows: null pointer argument");
  MOE_CHECK_ARG(aligned16(src) && aligned16(dst), "moe_gather_rows: pointers must be 16-byte aligned");
  MOE_CHECK_ARG(src_rows >= 0 && padded_rows > 0 && div > 0, "moe_gather_rows: bad sizes");
  MOE_ROW_COMMON_CHECKS("moe_gather_rows", cols, dtype);
  gather_rows_kernel<<<row_grid(padded_rows), kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), row_src, num_mtiles, static_cast<uint4*>(dst), cols / 8, div);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_dispatch_rows(const void* src, const int32_t* dst_row, const int32_t* row_src,
                                 const int32_t* num_mtiles, void* dst, int64_t num_tokens, int topk,
                                 int64_t padded_rows, int cols, int dtype, void* stream) {
  MOE_CHECK_ARG(num_tokens >= 0 && topk > 0 && padded_rows > 0, "moe_dispatch_rows: bad sizes");
  MOE_CHECK_ARG(src && dst_row && row_src && num_mtiles && dst, "moe_dispatch_rows: null pointer argument");
  MOE_CHECK_ARG(aligned16(src) && aligned16(dst), "moe_dispatch_rows: pointers must be 16-byte aligned");
  MOE_ROW_COMMON_CHECKS("moe_dispatch_rows", cols, dtype);
  const int token_blocks = row_grid(num_tokens);
  const int pad_blocks = sm_count();
  dispatch_rows_kernel<<<token_blocks + pad_blocks, kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), dst_row, row_src, num_mtiles, static_cast<uint4*>(dst), num_tokens, topk, cols / 8,
      token_blocks);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_gather_rows_peer(const void* const* peer_bases, const int32_t* src_rank, const int32_t* src_row,
                                    const float* scale, const int32_t* num_mtiles, const int32_t* tile_pairs,
                                    int num_experts, int chunk_index, int chunk_count, int pair_begin, int pair_end,
                                    void* dst, int64_t padded_rows, int cols, int dtype, int bulk_ctas,
                                    int dedicated_ctas, int32_t* status, void* stream) {
  MOE_CHECK_ARG(peer_bases && src_rank && src_row && num_mtiles && dst, "moe_gather_rows_peer: null pointer argument");
  MOE_CHECK_ARG(aligned16(dst), "moe_gather_rows_peer: dst must be 16-byte aligned");
  MOE_CHECK_ARG(padded_rows > 0, "moe_gather_rows_peer: bad sizes");
  MOE_CHECK_ARG((chunk_count >= 0 && chunk_count <= 1) ||
                    (tile_pairs != nullptr && num_experts > 0 && chunk_index >= 0 &&
                     (chunk_count > 1 ? chunk_index < chunk_count : chunk_index < -chunk_count && chunk_index < num_experts)),
                "moe_gather_rows_peer: chunk %d of %d needs tile_pairs, num_experts and a valid slice", chunk_index,
                chunk_count);
  MOE_CHECK_ARG(pair_end <= pair_begin || (tile_pairs != nullptr && pair_begin >= 0),
                "moe_gather_rows_peer: the pair range [%d, %d) needs tile_pairs and begin >= 0", pair_begin, pair_end);
  const RowWindow window{chunk_index, chunk_count, pair_begin, pair_end};
  const int mtiles_bound = static_cast<int>(padded_rows / MOE_TILE_M);
  MOE_ROW_COMMON_CHECKS("moe_gather_rows_peer", cols, dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* const* bases = reinterpret_cast<const uint4* const*>(peer_bases);
  if (bulk_ctas > 0) {
    // copy-engine variant: one row slot per warp, as many warps as 200 KB of shared memory hold (4..16)
    const size_t row_bytes = static_cast<size_t>(cols) * 2;
    int warps = static_cast<int>((200 * 1024) / row_bytes);
    if (warps > kBulkMaxWarps) warps = kBulkMaxWarps;
    if (warps >= 4) {
      const size_t smem = row_bytes * warps;
      const int grid_b = bulk_ctas < sm_count() ? bulk_ctas : sm_count();
      if (dtype == MOE_DTYPE_BF16) {
        MOE_CUDA(cudaFuncSetAttribute(pull_rows_bulk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        pull_rows_bulk_kernel<__nv_bfloat16><<<grid_b, warps * 32, smem, s>>>(
            bases, src_rank, src_row, scale, num_mtiles, tile_pairs, num_experts, mtiles_bound, window,
            static_cast<uint4*>(dst), cols / 8, wait_limit_cycles(), status);
      } else {
        MOE_CUDA(cudaFuncSetAttribute(pull_rows_bulk_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        pull_rows_bulk_kernel<__half><<<grid_b, warps * 32, smem, s>>>(
            bases, src_rank, src_row, scale, num_mtiles, tile_pairs, num_experts, mtiles_bound, window,
            static_cast<uint4*>(dst), cols / 8, wait_limit_cycles(), status);
      }
      MOE_CUDA(cudaGetLastError());
      return MOE_OK;
    }
    // rows too long for a slot: fall through to the load/store kernel
  }
  if (dedicated_ctas > 0) {
    // load/store kernel, one 1024-thread CTA on each SM the caller keeps free of GEMM CTAs
    const int grid_d = dedicated_ctas < sm_count() ? dedicated_ctas : sm_count();
    if (dtype == MOE_DTYPE_BF16) {
      gather_rows_peer_kernel<__nv_bfloat16, 1024><<<grid_d, 1024, 0, s>>>(bases, src_rank, src_row, scale, num_mtiles,
                                                                         tile_pairs, num_experts, mtiles_bound, window, static_cast<uint4*>(dst), cols / 8);
    } else {
      gather_rows_peer_kernel<__half, 1024><<<grid_d, 1024, 0, s>>>(bases, src_rank, src_row, scale, num_mtiles, tile_pairs,
                                                                  num_experts, mtiles_bound, window,
                                                                  static_cast<uint4*>(dst), cols / 8);
    }
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
  }
  // The load/store kernel spread over all SMs: bound by NVLink, not by SMs; small CTAs keep the links busy and one of
  // them still fits beside a grouped-GEMM CTA.
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int grid = static_cast<int>(padded_rows < cap ? padded_rows : cap);
  if (dtype == MOE_DTYPE_BF16) {
    gather_rows_peer_kernel<__nv_bfloat16, 128><<<grid, 128, 0, s>>>(bases, src_rank, src_row, scale, num_mtiles,
                                                                    tile_pairs, num_experts, mtiles_bound, window, static_cast<uint4*>(dst), cols / 8);
  } else {
    gather_rows_peer_kernel<__half, 128><<<grid, 128, 0, s>>>(bases, src_rank, src_row, scale, num_mtiles, tile_pairs,
                                                             num_experts, mtiles_bound, window,
                                                             static_cast<uint4*>(dst), cols / 8);
  }
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_unpad_rows(const void* src, const int32_t* dst_row, void* out, int64_t num_rows, int cols, int dtype,
                              void* stream) {
  MOE_CHECK_ARG(num_rows >= 0, "moe_unpad_rows: num_rows is negative");
  if (num_rows == 0) return MOE_OK;
  MOE_CHECK_ARG(src && dst_row && out, "moe_unpad_rows: null pointer argument");
  MOE_CHECK_ARG(aligned16(src) && aligned16(out), "moe_unpad_rows: pointers must be 16-byte aligned");
  MOE_ROW_COMMON_CHECKS("moe_unpad_rows", cols, dtype);
  unpad_rows_kernel<<<row_grid(num_rows), kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), dst_row, static_cast<uint4*>(out), num_rows, cols / 8);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_combine_topk(const void* ys, const void* scores, const int32_t* dst_row, void* out,
                                int64_t num_tokens, int topk, int cols, int dtype, void* stream) {
  MOE_CHECK_ARG(num_tokens >= 0 && topk > 0, "moe_combine_topk: bad sizes T=%lld topk=%d", (long long)num_tokens, topk);
  if (num_tokens == 0) return MOE_OK;
  MOE_CHECK_ARG(ys && dst_row && out, "moe_combine_topk: null pointer argument");
  MOE_CHECK_ARG(aligned16(ys) && aligned16(out), "moe_combine_topk: pointers must be 16-byte aligned");
  MOE_ROW_COMMON_CHECKS("moe_combine_topk", cols, dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = row_grid(num_tokens);
  if (dtype == MOE_DTYPE_BF16) {
    combine_topk_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, s>>>(
        static_cast<const uint4*>(ys), static_cast<const __nv_bfloat16*>(scores), dst_row, static_cast<uint4*>(out),
        num_tokens, topk, cols / 8);
  } else {
    combine_topk_kernel<__half><<<grid, kRowThreads, 0, s>>>(static_cast<const uint4*>(ys),
                                                             static_cast<const __half*>(scores), dst_row,
                                                             static_cast<uint4*>(out), num_tokens, topk, cols / 8);
  }
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

extern "C" int moe_combine_bwd(const void* dout, const void* scores, const void* ys, const int32_t* row_src,
                               const int32_t* num_mtiles, void* gs, void* dscores, int64_t num_tokens, int topk,
                               int64_t padded_rows, int cols, int dtype, void* stream) {
  MOE_CHECK_ARG(dout && scores && ys && row_src && num_mtiles && dscores, "moe_combine_bwd: null pointer argument");
  MOE_CHECK_ARG(aligned16(dout) && aligned16(ys) && aligned16(gs), "moe_combine_bwd: pointers must be 16-byte aligned");
  MOE_CHECK_ARG(num_tokens >= 0 && topk > 0 && padded_rows > 0, "moe_combine_bwd: bad sizes");
  MOE_ROW_COMMON_CHECKS("moe_combine_bwd", cols, dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = row_grid((padded_rows + kRowThreads / 32 - 1) / (kRowThreads / 32));
  if (dtype == MOE_DTYPE_BF16) {
    combine_bwd_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, s>>>(
        static_cast<const uint4*>(dout), static_cast<const __nv_bfloat16*>(scores), static_cast<const uint4*>(ys),
        row_src, num_mtiles, static_cast<uint4*>(gs), static_cast<__nv_bfloat16*>(dscores), topk, cols / 8);
  } else {
    combine_bwd_kernel<__half><<<grid, kRowThreads, 0, s>>>(
        static_cast<const uint4*>(dout), static_cast<const __half*>(scores), static_cast<const uint4*>(ys), row_src,
        num_mtiles, static_cast<uint4*>(gs), static_cast<__half*>(dscores), topk, cols / 8);
  }
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

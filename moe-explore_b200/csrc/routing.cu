// Routing metadata: per-expert histogram, prefix sums, STABLE permutation by expert and its
// inverse, plus the padded expert-sorted row layout the grouped GEMMs consume.
//
// Replaces get_token_indices (reference: src/moe_explore/expert_permute.py:19-41), which runs
// torch.argsort + torch.histc + torch.cumsum as three or more launches.  Here it is a
// three-kernel counting sort (the number of distinct keys, E, is small):
//   1. chunk_histogram : each warp owns a contiguous chunk of kChunk flat positions and counts
//                        its ids per expert in shared memory (warp-aggregated via match.any);
//   2. scan_offsets    : turns the [chunks, E] histogram into per-(chunk, expert) exclusive
//                        offsets (one CTA per expert scans down the chunk axis when there are many
//                        chunks), then one CTA derives the per-expert prefix sums (unpadded and
//                        padded to 128-row tiles) and the tile -> expert map;
//   3. place_rows      : each warp walks its chunk again in order, ranks equal ids with
//                        match.any + popc (which preserves flat-position order) and writes
//                        perm / row_src / dst_row.
// All arithmetic is integer; results are bit-exact with torch.sort(stable=True).
// HBM traffic: 2 x 8R bytes read (ids, twice) + 8R (perm) + 4R (dst_row) + 4RP (row_src) written.
#include "common.cuh"

namespace moe {

constexpr int kChunk = 1024;        // flat positions per warp
constexpr int kWarpsPerBlock = 8;
constexpr int kMaxExperts = 1024;   // scan kernel uses one thread per expert

__host__ __device__ inline int64_t num_chunks(int64_t R) { return (R + kChunk - 1) / kChunk; }

// Peers of this lane holding the same key (full-warp, inactive lanes pass key = -1 - lane so they match nobody).
__device__ __forceinline__ unsigned match_key(int key) { return __match_any_sync(0xFFFFFFFFu, key); }

// Lane `lane` of the warp that owns [begin, begin + kChunk) loads its 32 ids (positions begin + 32*i + lane)
// with independent loads so their latencies overlap.  Positions past R and ids outside [0, E) become
// negative keys that match no other lane.
__device__ __forceinline__ void load_keys(const int64_t* __restrict__ ids, int64_t begin, int64_t R, int E, int lane,
                                          int (&keys)[kChunk / 32], int32_t* status) {
  int64_t raw[kChunk / 32];
#pragma unroll
  for (int i = 0; i < kChunk / 32; ++i) {
    const int64_t j = begin + 32 * i + lane;
    raw[i] = j < R ? ids[j] : -1;
  }
  bool bad = false;
#pragma unroll
  for (int i = 0; i < kChunk / 32; ++i) {
    const int64_t j = begin + 32 * i + lane;
    const bool ok = raw[i] >= 0 && raw[i] < E;
    bad |= (j < R) && !ok;
    keys[i] = ok ? static_cast<int>(raw[i]) : -1 - lane;
  }
  if (bad && status != nullptr) atomicCAS(status, 0, DS_BAD_EXPERT_ID);  // id out of range: dropped from every output
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
chunk_histogram_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int32_t* __restrict__ chunk_hist,
                       int32_t* status) {
  extern __shared__ int32_t sh_cnt[];  // [kWarpsPerBlock][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* cnt = sh_cnt + warp * E;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  const int64_t begin = chunk * kChunk;
  if (begin >= R) return;
  int keys[kChunk / 32];
  load_keys(ids, begin, R, E, lane, keys, status);
#pragma unroll
  for (int i = 0; i < kChunk / 32; ++i) {
    const int key = keys[i];
    const unsigned peers = match_key(key);
    if (key >= 0 && (peers & ((1u << lane) - 1)) == 0) cnt[key] += __popc(peers);  // lowest peer adds for the group
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32) chunk_hist[chunk * E + e] = cnt[e];
}

// Pair entry layout: bits 0-19 first tile, bits 20-30 expert, bit 31 "the pair has a second tile"
// (so one load tells a CTA pair everything about its next work item).  The per-expert exclusive prefix of
// the pair counts follows the pair list in the same buffer, at index `mtiles_bound` ([E+1] entries).
// Tile -> expert map and the pair list for expert e, whose padded rows start at `row_begin` and span
// `padded` rows; its pairs start at index `pair_begin`.
__device__ __forceinline__ void write_tile_maps(int e, int32_t row_begin, int32_t padded, int32_t pair_begin,
                                                int32_t* __restrict__ mtile_expert, int32_t* __restrict__ tile_pairs,
                                                int32_t* __restrict__ pair_prefix) {
  const int first = row_begin / MOE_TILE_M;
  const int last = first + padded / MOE_TILE_M;
  for (int m = first; m < last; ++m) mtile_expert[m] = e;
  if (tile_pairs != nullptr) {
    pair_prefix[e] = pair_begin;  // exclusive prefix of pair counts: expert e's pairs are [prefix[e], prefix[e+1])
    for (int m = first, p = pair_begin; m < last; m += 2, ++p)
      tile_pairs[p] = static_cast<int32_t>(static_cast<uint32_t>(m) | (static_cast<uint32_t>(e) << 20) |
                                           (m + 1 < last ? 0x80000000u : 0u));
  }
}

// Many chunks: one CTA per expert turns its column of the [chunks, E] histogram into exclusive offsets (every
// thread owns a contiguous run of chunks; block-wide scan of the run sums) and leaves the expert's row count in
// group_indices[e + 1] for the single-CTA pass below.
constexpr int kScanThreads = 256;
__global__ void __launch_bounds__(kScanThreads)
scan_chunks_kernel(const int32_t* __restrict__ chunk_hist, int32_t* __restrict__ chunk_off, int64_t nchunks, int E,
                   int32_t* __restrict__ group_indices) {
  __shared__ int32_t warp_sum[kScanThreads / 32];
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t per = (nchunks + kScanThreads - 1) / kScanThreads;
  const int64_t c0 = tid * per;
  const int64_t c1 = c0 + per < nchunks ? c0 + per : nchunks;
  int32_t mine = 0;
  for (int64_t c = c0; c < c1; ++c) mine += chunk_hist[c * E + e];
  int32_t incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  int32_t before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kScanThreads / 32; ++w) {
    if (w < warp) before += warp_sum[w];
    total += warp_sum[w];
  }
  int32_t run = before + incl - mine;
  for (int64_t c = c0; c < c1; ++c) {
    chunk_off[c * E + e] = run;
    run += chunk_hist[c * E + e];
  }
  if (tid == 0) group_indices[e + 1] = total;
}

// One CTA, one thread per expert (E <= 1024).  `counts_ready`: the per-expert row counts are already in
// group_indices[1..E] (scan_chunks_kernel ran); otherwise this kernel scans the chunk axis itself (few chunks).
// num_mtiles receives {tiles in use, tile pairs in use, mtiles_bound, 0}; perm entries past the rows that were
// kept (ids out of range are dropped) are set to -1.
__global__ void __launch_bounds__(kMaxExperts)
scan_offsets_kernel(const int32_t* __restrict__ chunk_hist, int32_t* __restrict__ chunk_off, int64_t nchunks, int E,
                    int counts_ready, int32_t* __restrict__ group_indices,
                    int32_t* __restrict__ pad_offsets, int32_t* __restrict__ mtile_expert,
                    int32_t* __restrict__ tile_pairs, int32_t* __restrict__ num_mtiles, int mtiles_bound,
                    int64_t* __restrict__ perm, int64_t R) {
  __shared__ int32_t sh_a[kMaxExperts];
  __shared__ int32_t sh_b[kMaxExperts];
  __shared__ int32_t sh_c[kMaxExperts];
  const int e = threadIdx.x;
  int32_t total = 0;
  if (e < E) {
    if (counts_ready) {
      total = group_indices[e + 1];
    } else {
      // exclusive scan down the chunk axis for this expert
      constexpr int kBatch = 16;  // loads in flight per thread
      for (int64_t c0 = 0; c0 < nchunks; c0 += kBatch) {
        int32_t v[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) v[i] = (c0 + i < nchunks) ? chunk_hist[(c0 + i) * E + e] : 0;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          if (c0 + i < nchunks) chunk_off[(c0 + i) * E + e] = total;
          total += v[i];
        }
      }
    }
  }
  const int32_t padded = (total + MOE_TILE_M - 1) / MOE_TILE_M * MOE_TILE_M;
  const int32_t pairs = (padded / MOE_TILE_M + 1) / 2;  // row tiles of one expert, two at a time
  sh_a[e] = e < E ? total : 0;
  sh_b[e] = e < E ? padded : 0;
  sh_c[e] = e < E ? pairs : 0;
  __syncthreads();
  // Hillis-Steele inclusive scan over experts for the three sequences.
  for (int off = 1; off < kMaxExperts; off <<= 1) {
    int32_t a = 0, b = 0, c = 0;
    if (e >= off) { a = sh_a[e - off]; b = sh_b[e - off]; c = sh_c[e - off]; }
    __syncthreads();
    sh_a[e] += a;
    sh_b[e] += b;
    sh_c[e] += c;
    __syncthreads();
  }
  if (e < E) {
    group_indices[e + 1] = sh_a[e];
    pad_offsets[e + 1] = sh_b[e];
    if (e == 0) { group_indices[0] = 0; pad_offsets[0] = 0; }
    int32_t* pair_prefix = tile_pairs != nullptr ? tile_pairs + mtiles_bound : nullptr;
    if (mtile_expert != nullptr) write_tile_maps(e, sh_b[e] - padded, padded, sh_c[e] - pairs, mtile_expert, tile_pairs, pair_prefix);
    if (num_mtiles != nullptr && e == E - 1) {
      num_mtiles[0] = sh_b[e] / MOE_TILE_M;
      num_mtiles[1] = sh_c[e];
      num_mtiles[2] = mtiles_bound;
      num_mtiles[3] = 0;
      if (pair_prefix != nullptr) pair_prefix[E] = sh_c[e];
    }
  }
  if (perm != nullptr) {
    const int64_t kept = sh_a[E - 1];
    for (int64_t r = kept + threadIdx.x; r < R; r += kMaxExperts) perm[r] = -1;
  }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
place_rows_kernel(const int64_t* __restrict__ ids, int64_t R, int E, const int32_t* __restrict__ chunk_off,
                  const int32_t* __restrict__ group_indices, const int32_t* __restrict__ pad_offsets,
                  int64_t* __restrict__ perm, int32_t* __restrict__ row_src, int32_t* __restrict__ dst_row) {
  extern __shared__ int32_t sh_cnt[];  // [kWarpsPerBlock][E]: rank of the next row of expert e inside the expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* cnt = sh_cnt + warp * E;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  const int64_t begin = chunk * kChunk;
  if (begin >= R) return;
  for (int e = lane; e < E; e += 32) cnt[e] = chunk_off[chunk * E + e];
  __syncwarp();
  int keys[kChunk / 32];
  load_keys(ids, begin, R, E, lane, keys, nullptr);
#pragma unroll
  for (int i = 0; i < kChunk / 32; ++i) {
    const int key = keys[i];
    const int64_t j = begin + 32 * i + lane;
    const unsigned peers = match_key(key);
    const unsigned before = peers & ((1u << lane) - 1);
    int32_t rank = 0;
    if (key >= 0) rank = cnt[key] + __popc(before);  // lanes are in flat-position order: stable
    __syncwarp();
    if (key >= 0 && before == 0) cnt[key] += __popc(peers);
    __syncwarp();
    if (key >= 0) {
      if (perm != nullptr) perm[group_indices[key] + rank] = j;
      const int32_t p = pad_offsets[key] + rank;
      if (row_src != nullptr) row_src[p] = static_cast<int32_t>(j);
      if (dst_row != nullptr) dst_row[j] = p;
    } else if (j < R && dst_row != nullptr) {
      dst_row[j] = -1;  // id out of range: the row is in no expert's segment; consumers skip negative rows
    }
  }
}

// Layout from an existing exclusive prefix (rows already grouped): one CTA, thread per expert for
// the padded prefix, then all threads fill the row maps.
__global__ void __launch_bounds__(kMaxExperts)
layout_from_groups_kernel(const int32_t* __restrict__ group_indices, int64_t R, int E, int32_t* __restrict__ pad_offsets,
                          int32_t* __restrict__ mtile_expert, int32_t* __restrict__ tile_pairs,
                          int32_t* __restrict__ num_mtiles, int mtiles_bound, int32_t* status) {
  __shared__ int32_t sh_b[kMaxExperts];
  __shared__ int32_t sh_c[kMaxExperts];
  const int e = threadIdx.x;
  int32_t padded = 0;
  if (e < E) {
    // a prefix that is not monotone, does not start at 0 or does not end at R describes no layout: such experts
    // get no rows here and the status word says so
    const int32_t lo = group_indices[e], hi = group_indices[e + 1];
    const bool bad = hi < lo || lo < 0 || hi > R || (e == 0 && lo != 0) || (e == E - 1 && hi != R);
    if (bad && status != nullptr) atomicCAS(status, 0, DS_BAD_LAYOUT);
    const int32_t cnt = bad ? 0 : hi - lo;
    padded = (cnt + MOE_TILE_M - 1) / MOE_TILE_M * MOE_TILE_M;
  }
  const int32_t pairs = (padded / MOE_TILE_M + 1) / 2;
  sh_b[e] = padded;
  sh_c[e] = pairs;
  __syncthreads();
  for (int off = 1; off < kMaxExperts; off <<= 1) {
    int32_t b = 0, c = 0;
    if (e >= off) { b = sh_b[e - off]; c = sh_c[e - off]; }
    __syncthreads();
    sh_b[e] += b;
    sh_c[e] += c;
    __syncthreads();
  }
  if (e < E) {
    pad_offsets[e + 1] = sh_b[e];
    if (e == 0) pad_offsets[0] = 0;
    int32_t* pair_prefix = tile_pairs != nullptr ? tile_pairs + mtiles_bound : nullptr;
    if (mtile_expert != nullptr) write_tile_maps(e, sh_b[e] - padded, padded, sh_c[e] - pairs, mtile_expert, tile_pairs, pair_prefix);
    if (num_mtiles != nullptr && e == E - 1) {
      num_mtiles[0] = sh_b[e] / MOE_TILE_M;
      num_mtiles[1] = sh_c[e];
      num_mtiles[2] = mtiles_bound;
      num_mtiles[3] = 0;
      if (pair_prefix != nullptr) pair_prefix[E] = sh_c[e];
    }
  }
}

__global__ void layout_rows_kernel(const int32_t* __restrict__ group_indices, const int32_t* __restrict__ pad_offsets,
                                   int64_t R, int E, int32_t* __restrict__ row_src, int32_t* __restrict__ dst_row) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= R) return;
  // binary search: largest e with group_indices[e] <= j
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (group_indices[mid] <= j) lo = mid; else hi = mid;
  }
  // rows of a segment the layout kernel refused (bad prefix) have no padded row
  const int64_t in_seg = j - group_indices[lo];
  const bool ok = in_seg >= 0 && in_seg < pad_offsets[lo + 1] - pad_offsets[lo] && j < group_indices[lo + 1];
  const int32_t p = ok ? pad_offsets[lo] + static_cast<int32_t>(in_seg) : -1;
  if (ok && row_src != nullptr) row_src[p] = static_cast<int32_t>(j);
  if (dst_row != nullptr) dst_row[j] = p;
}

}  // namespace moe

using namespace moe;

extern "C" int64_t moe_padded_rows_bound(int64_t num_rows, int num_experts) {
  if (num_rows < 0 || num_experts <= 0) return 0;
  // sum over experts of ceil(c_e / 128) * 128 <= R + E * 127, rounded up to a tile
  const int64_t worst = num_rows + static_cast<int64_t>(num_experts) * (MOE_TILE_M - 1);
  const int64_t rp = (worst + MOE_TILE_M - 1) / MOE_TILE_M * MOE_TILE_M;
  return rp > 0 ? rp : MOE_TILE_M;
}

extern "C" int64_t moe_mtiles_bound(int64_t num_rows, int num_experts) {
  return moe_padded_rows_bound(num_rows, num_experts) / MOE_TILE_M;
}

extern "C" size_t moe_routing_workspace_bytes(int64_t num_rows, int num_experts) {
  if (num_rows < 0 || num_experts <= 0) return 0;
  const int64_t chunks = num_chunks(num_rows) > 0 ? num_chunks(num_rows) : 1;
  return 2 * static_cast<size_t>(chunks) * num_experts * sizeof(int32_t);  // chunk histogram + chunk offsets
}

extern "C" int moe_routing_metadata(const int64_t* expert_idx, int64_t num_rows, int num_experts,
                                    int32_t* group_indices, int64_t* perm, int32_t* pad_offsets, int32_t* row_src,
                                    int32_t* dst_row, int32_t* mtile_expert, int32_t* tile_pairs,
                                    int32_t* num_mtiles, int32_t* status, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  MOE_CHECK_ARG(num_rows >= 0, "moe_routing_metadata: num_rows=%lld is negative", (long long)num_rows);
  MOE_CHECK_ARG(num_experts > 0, "moe_routing_metadata: num_experts=%d must be positive", num_experts);
  if (num_experts > kMaxExperts) {
    set_error("moe_routing_metadata: num_experts=%d exceeds the supported maximum %d", num_experts, kMaxExperts);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(moe_mtiles_bound(num_rows, num_experts) < (1ll << 20),
                "moe_routing_metadata: num_rows=%lld needs more than 2^20 row tiles", (long long)num_rows);
  MOE_CHECK_ARG(group_indices && pad_offsets, "moe_routing_metadata: group_indices and pad_offsets are required");
  MOE_CHECK_ARG(num_rows == 0 || expert_idx != nullptr, "moe_routing_metadata: expert_idx is null");
  MOE_CHECK_ARG((mtile_expert == nullptr) == (num_mtiles == nullptr) && (tile_pairs == nullptr || mtile_expert != nullptr),
                "moe_routing_metadata: mtile_expert, tile_pairs and num_mtiles go together");
  MOE_CHECK_ARG(workspace != nullptr && workspace_bytes >= moe_routing_workspace_bytes(num_rows, num_experts),
                "moe_routing_metadata: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
                moe_routing_workspace_bytes(num_rows, num_experts));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* chunk_hist = static_cast<int32_t*>(workspace);
  const int64_t chunks = num_chunks(num_rows);
  int32_t* chunk_off = chunk_hist + (chunks > 0 ? chunks : 1) * num_experts;
  const int blocks = static_cast<int>((chunks + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t sh = static_cast<size_t>(kWarpsPerBlock) * num_experts * sizeof(int32_t);
  if (row_src != nullptr) {
    MOE_CUDA(cudaMemsetAsync(row_src, 0xFF, moe_padded_rows_bound(num_rows, num_experts) * sizeof(int32_t), s));
  }
  if (chunks == 0) {
    MOE_CUDA(cudaMemsetAsync(chunk_hist, 0, num_experts * sizeof(int32_t), s));
  } else {
    chunk_histogram_kernel<<<blocks, kWarpsPerBlock * 32, sh, s>>>(expert_idx, num_rows, num_experts, chunk_hist, status);
    MOE_CUDA(cudaGetLastError());
  }
  // many chunks: scan the chunk axis with one CTA per expert first (a single CTA walking 512 chunks took 53 us)
  const int split_scan = chunks > 64 ? 1 : 0;
  if (split_scan) {
    scan_chunks_kernel<<<num_experts, kScanThreads, 0, s>>>(chunk_hist, chunk_off, chunks, num_experts, group_indices);
    MOE_CUDA(cudaGetLastError());
  }
  scan_offsets_kernel<<<1, kMaxExperts, 0, s>>>(chunk_hist, chunk_off, chunks, num_experts, split_scan, group_indices,
                                               pad_offsets, mtile_expert, tile_pairs, num_mtiles,
                                               static_cast<int>(moe_mtiles_bound(num_rows, num_experts)), perm, num_rows);
  MOE_CUDA(cudaGetLastError());
  if (chunks > 0 && (perm || row_src || dst_row)) {
    place_rows_kernel<<<blocks, kWarpsPerBlock * 32, sh, s>>>(expert_idx, num_rows, num_experts, chunk_off,
                                                             group_indices, pad_offsets, perm, row_src, dst_row);
    MOE_CUDA(cudaGetLastError());
  }
  return MOE_OK;
}

extern "C" int moe_layout_from_groups(const int32_t* group_indices, int64_t num_rows, int num_experts,
                                      int32_t* pad_offsets, int32_t* row_src, int32_t* dst_row, int32_t* mtile_expert,
                                      int32_t* tile_pairs, int32_t* num_mtiles, int32_t* status, void* stream) {
  MOE_CHECK_ARG(group_indices && pad_offsets, "moe_layout_from_groups: group_indices and pad_offsets are required");
  MOE_CHECK_ARG(num_rows >= 0 && num_experts > 0, "moe_layout_from_groups: bad sizes R=%lld E=%d", (long long)num_rows,
                num_experts);
  MOE_CHECK_ARG(moe_mtiles_bound(num_rows, num_experts) < (1ll << 20),
                "moe_layout_from_groups: num_rows=%lld needs more than 2^20 row tiles", (long long)num_rows);
  if (num_experts > kMaxExperts) {
    set_error("moe_layout_from_groups: num_experts=%d exceeds the supported maximum %d", num_experts, kMaxExperts);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG((mtile_expert == nullptr) == (num_mtiles == nullptr) && (tile_pairs == nullptr || mtile_expert != nullptr),
                "moe_layout_from_groups: mtile_expert, tile_pairs and num_mtiles go together");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row_src != nullptr) {
    MOE_CUDA(cudaMemsetAsync(row_src, 0xFF, moe_padded_rows_bound(num_rows, num_experts) * sizeof(int32_t), s));
  }
  layout_from_groups_kernel<<<1, kMaxExperts, 0, s>>>(group_indices, num_rows, num_experts, pad_offsets, mtile_expert,
                                                     tile_pairs, num_mtiles,
                                                     static_cast<int>(moe_mtiles_bound(num_rows, num_experts)), status);
  MOE_CUDA(cudaGetLastError());
  if (num_rows > 0 && (row_src || dst_row)) {
    const int threads = 256;
    const int blocks = static_cast<int>((num_rows + threads - 1) / threads);
    layout_rows_kernel<<<blocks, threads, 0, s>>>(group_indices, pad_offsets, num_rows, num_experts, row_src, dst_row);
    MOE_CUDA(cudaGetLastError());
  }
  return MOE_OK;
}

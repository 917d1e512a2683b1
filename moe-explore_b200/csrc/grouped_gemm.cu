// Host side of the grouped GEMMs: argument checks, tensor maps (cached), scheduling choices and the
// C entry points.  The kernel itself is in gemm_kernel.cuh; its variants are instantiated in gemm_inst_*.cu.
#include "gemm_kernel.cuh"

#include <mutex>

namespace moe {

#define MOE_EXTERN(T, CTAS, BN, A_K, B_K, EPI, KG, GATHER)                                                       \
  extern template int launch<T, BN, A_K, B_K, EPI, KG, CTAS, GATHER>(const CUtensorMap&, const CUtensorMap&,       \
                                                                     const CUtensorMap&, const CUtensorMap&, GemmArgs, \
                                                                     const LaunchParams&);
// every variant without the row gather; with it, the variants the gathering entry points reach
#define MOE_EXTERN_BN(T, CTAS, BN)                                \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_ACT, false, false)     \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_GLU, false, false)     \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_ACT_AUX, false, false) \
  MOE_EXTERN(T, CTAS, BN, true, true, EPI_ACT, false, false)      \
  MOE_EXTERN(T, CTAS, BN, true, true, EPI_ACT_AUX, false, false)  \
  MOE_EXTERN(T, CTAS, BN, true, true, EPI_DGLU, false, false)     \
  MOE_EXTERN(T, CTAS, BN, false, false, EPI_ACT, true, false)     \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_ACT, false, true)      \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_GLU, false, true)      \
  MOE_EXTERN(T, CTAS, BN, true, false, EPI_ACT_AUX, false, true)  \
  MOE_EXTERN(T, CTAS, BN, true, true, EPI_ACT, false, true)       \
  MOE_EXTERN(T, CTAS, BN, true, true, EPI_ACT_AUX, false, true)   \
  MOE_EXTERN(T, CTAS, BN, false, false, EPI_ACT, true, true)
#define MOE_EXTERN_ALL(T, CTAS) MOE_EXTERN_BN(T, CTAS, 128) MOE_EXTERN_BN(T, CTAS, 256)
MOE_EXTERN_ALL(__nv_bfloat16, 2)
MOE_EXTERN_ALL(__nv_bfloat16, 1)
MOE_EXTERN_ALL(__half, 2)
MOE_EXTERN_ALL(__half, 1)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
      cached.store(fn, std::memory_order_release);
    }
  }
  return fn;
}

// Tensor maps depend only on (address, element type, extents, box), never on the data, so they are kept: a training
// step encodes the same dozen maps again and again (a few microseconds each, which is what small token counts
// are bound by).  A small table with round-robin replacement, shared by all threads.
struct TmapKey {
  const void* ptr;
  int dtype;
  int rank;
  uint64_t dims[4];
  uint64_t strides[3];  // bytes, of dims 1..rank-1
  uint32_t box[4];
  bool operator==(const TmapKey& o) const {
    if (ptr != o.ptr || dtype != o.dtype || rank != o.rank) return false;
    for (int i = 0; i < rank; ++i)
      if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
    for (int i = 0; i + 1 < rank; ++i)
      if (strides[i] != o.strides[i]) return false;
    return true;
  }
};
constexpr int kTmapCacheSize = 128;
static std::mutex g_tmap_mutex;
static TmapKey g_tmap_keys[kTmapCacheSize];
static CUtensorMap g_tmap_vals[kTmapCacheSize];
static int g_tmap_used = 0, g_tmap_next = 0;

// Tensor map with the 128-byte swizzle; dims[0] is the contiguous dimension.  `strides` (bytes, for dims 1..rank-1)
// may be null for a dense row-major tensor.
static int make_tmap(CUtensorMap* map, int dtype, const void* ptr, int rank, const uint64_t* dims,
                     const uint32_t* box, const uint64_t* strides = nullptr) {
  TmapKey key{};
  key.ptr = ptr;
  key.dtype = dtype;
  key.rank = rank;
  uint64_t dense = 2;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    dense *= dims[i];
    if (i < rank - 1) key.strides[i] = strides != nullptr ? strides[i] : dense;
  }
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    for (int i = 0; i < g_tmap_used; ++i)
      if (g_tmap_keys[i] == key) {
        *map = g_tmap_vals[i];
        return MOE_OK;
      }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return MOE_ERR_CUDA;
  }
  cuuint64_t gdim[4];
  cuuint64_t gstride[3];
  cuuint32_t bdim[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    if (i < rank - 1) gstride[i] = key.strides[i];
  }
  CUresult r = fn(map, dtype == MOE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  rank, const_cast<void*>(ptr), gdim, gstride, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu x %llu)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1),
              (unsigned long long)(rank > 2 ? dims[2] : 1));
    return MOE_ERR_CUDA;
  }
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    const int slot = g_tmap_used < kTmapCacheSize ? g_tmap_used++ : (g_tmap_next++ % kTmapCacheSize);
    g_tmap_keys[slot] = key;
    g_tmap_vals[slot] = *map;
  }
  return MOE_OK;
}

// Blocked view of a [rows, cols] (x batch) matrix whose contiguous extent is a multiple of 64 elements:
// dims {64, rows, cols / 64 (, batch)}, so that ONE copy with a {64, box_rows, blocks} box fetches `blocks` adjacent
// 64-column blocks, each landing as a box_rows x 128-byte swizzled tile (the layout of separate 64-wide copies).
static int make_tmap_blocked(CUtensorMap* map, int dtype, const void* ptr, uint64_t rows, uint64_t cols, uint64_t batch,
                             uint32_t box_rows, uint32_t blocks) {
  const uint64_t dims[4] = {64, rows, cols / 64, batch};
  const uint64_t strides[3] = {cols * 2, 128, rows * cols * 2};
  const uint32_t box[4] = {64, box_rows, blocks, 1};
  return make_tmap(map, dtype, ptr, batch > 0 ? 4 : 3, dims, box, strides);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Arrival counters of the wave barrier for callers that do not bring their own: a small ring in device memory;
// every launch that uses the barrier takes the next slot and zeroes it on its stream first.  A slot that another
// launch re-zeroes under a running kernel only costs that kernel its barrier (it falls back to the static stride).
constexpr int kWaveSlots = 256;
static __device__ uint32_t g_wave_counters[kWaveSlots];

static int ring_wave_counter(uint32_t** out) {
  static std::atomic<uint32_t*> base[64];
  static std::atomic<unsigned> next{0};
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  uint32_t* b = (dev >= 0 && dev < 64) ? base[dev].load(std::memory_order_acquire) : nullptr;
  if (b == nullptr) {
    void* p = nullptr;
    MOE_CUDA(cudaGetSymbolAddress(&p, g_wave_counters));
    b = static_cast<uint32_t*>(p);
    if (dev >= 0 && dev < 64) base[dev].store(b, std::memory_order_release);
  }
  *out = b + (next.fetch_add(1, std::memory_order_relaxed) % kWaveSlots);
  return MOE_OK;
}

static moe_gemm_options resolve(const moe_gemm_options* o) {
  moe_gemm_options r{};
  if (o != nullptr) r = *o;
  return r;
}

// 256-column tiles whenever there is more than one 128-column tile of work: with CTA pairs a 256 x 128 x 16 MMA
// takes ~144 cycles against ~158 for 256 x 256 x 16 (its operand reads from shared memory are the limit), so a
// half-empty last 256-column tile is far cheaper than narrow tiles throughout.
static int pick_bn(int N) { return N <= 128 ? 128 : 256; }

// What an M-grouped call may add to the plain contraction.
struct MExtras {
  void* aux_out = nullptr;
  const void* aux_in = nullptr;
  void* const* push_bases = nullptr;   // EPI_ACT: rows go to other GPUs' buffers
  const int32_t* push_rank = nullptr;
  const int32_t* push_row = nullptr;
  const int32_t* gather_row_src = nullptr;  // A rows are gathered from a [gather_rows, K] tensor by the loads
  int gather_div = 1;
  int64_t gather_rows = 0;
  const int32_t* combine_row_src = nullptr;  // EPI_ACT: rows are scaled and added into token-order rows
  const void* combine_scores = nullptr;
  int combine_topk = 1;
  int chunk_index = 0;
  int chunk_count = 1;
};

template <typename T, int BN, int CTAS>
static int mgrouped_dispatch(const void* a, const void* w, int64_t a_rows, int K, int N, int E, int w_transposed, int epi,
                             const GemmArgs& args, int dtype, const LaunchParams& lp) {
  CUtensorMap ta, tb;
  const bool gather = args.a_row_src != nullptr;  // selects the kernel variant whose operand loads gather rows
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)a_rows};
    const uint32_t box[2] = {BK, args.a_row_src != nullptr ? 1u : (uint32_t)BM};
    int rc = make_tmap(&ta, dtype, a, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  if (w_transposed) {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)E};
    const uint32_t box[3] = {BK, (uint32_t)(BN / CTAS), 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  } else if (args.b_blocked) {
    int rc = make_tmap_blocked(&tb, dtype, w, (uint64_t)K, (uint64_t)N, (uint64_t)E, BK, (uint32_t)(BN / CTAS / 64));
    if (rc != MOE_OK) return rc;
  } else {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)E};
    const uint32_t box[3] = {64, BK, 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  }
  if (epi == EPI_ACT) {
    CUtensorMap td = ta;
    if (args.out_tma) {
      const uint64_t dims[2] = {(uint64_t)N, (uint64_t)(args.mtiles_bound) * BM};
      const uint32_t box[2] = {64, 32};
      int rc = make_tmap(&td, dtype, args.out, 2, dims, box);
      if (rc != MOE_OK) return rc;
    }
    if (gather)
      return w_transposed ? launch<T, BN, true, true, EPI_ACT, false, CTAS, true>(ta, tb, ta, td, args, lp)
                          : launch<T, BN, true, false, EPI_ACT, false, CTAS, true>(ta, tb, ta, td, args, lp);
    return w_transposed ? launch<T, BN, true, true, EPI_ACT, false, CTAS, false>(ta, tb, ta, td, args, lp)
                        : launch<T, BN, true, false, EPI_ACT, false, CTAS, false>(ta, tb, ta, td, args, lp);
  } else if (epi == EPI_GLU) {
    return gather ? launch<T, BN, true, false, EPI_GLU, false, CTAS, true>(ta, tb, ta, ta, args, lp)
                  : launch<T, BN, true, false, EPI_GLU, false, CTAS, false>(ta, tb, ta, ta, args, lp);
  } else if (epi == EPI_ACT_AUX) {
    if (gather)
      return w_transposed ? launch<T, BN, true, true, EPI_ACT_AUX, false, CTAS, true>(ta, tb, ta, ta, args, lp)
                          : launch<T, BN, true, false, EPI_ACT_AUX, false, CTAS, true>(ta, tb, ta, ta, args, lp);
    return w_transposed ? launch<T, BN, true, true, EPI_ACT_AUX, false, CTAS, false>(ta, tb, ta, ta, args, lp)
                        : launch<T, BN, true, false, EPI_ACT_AUX, false, CTAS, false>(ta, tb, ta, ta, args, lp);
  }
  // EPI_DGLU (always with the transposed weight: dAct = g @ W2^T): the saved product and the result are moved by
  // tensor copies of 32-row x 64-column boxes
  CUtensorMap tc, td;
  {
    const uint64_t dims[2] = {(uint64_t)(2 * N), (uint64_t)a_rows};
    const uint32_t box[2] = {64, 32};
    int rc = make_tmap(&tc, dtype, args.aux_in, 2, dims, box);
    if (rc != MOE_OK) return rc;
    rc = make_tmap(&td, dtype, args.out, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  return launch<T, BN, true, true, EPI_DGLU, false, CTAS, false>(ta, tb, tc, td, args, lp);
}

static int mgrouped_common(const char* name, const void* a, const void* w, void* out, const MExtras& x,
                           const int32_t* mtile_expert, const int32_t* tile_pairs, const int32_t* num_mtiles,
                           int64_t padded_rows, int K, int N, int E, int w_transposed, int epi, int act, int dtype,
                           const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(a && w && (out || x.push_bases) && mtile_expert && num_mtiles, "%s: null pointer argument", name);
  MOE_CHECK_ARG(aligned16(a) && aligned16(w) && aligned16(out) && aligned16(x.aux_out) && aligned16(x.aux_in),
                "%s: pointers must be 16-byte aligned", name);
  MOE_CHECK_ARG(padded_rows > 0 && padded_rows % BM == 0, "%s: padded_rows=%lld must be a positive multiple of %d", name,
                (long long)padded_rows, BM);
  MOE_CHECK_ARG(K > 0 && N > 0 && E > 0, "%s: K=%d N=%d E=%d must be positive", name, K, N, E);
  if (K % 8 != 0 || N % 8 != 0 || (epi == EPI_GLU && N % 16 != 0)) {
    set_error("%s: K=%d and N=%d must be multiples of 8 (16 for GLU outputs): rows must be 16-byte aligned", name, K, N);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(dtype == MOE_DTYPE_BF16 || dtype == MOE_DTYPE_F16, "%s: unknown dtype %d", name, dtype);
  MOE_CHECK_ARG(x.chunk_count <= 1 || (tile_pairs != nullptr && x.chunk_index >= 0 && x.chunk_index < x.chunk_count),
                "%s: chunk %d of %d needs tile_pairs and 0 <= index < count", name, x.chunk_index, x.chunk_count);
  MOE_CHECK_ARG(x.gather_row_src == nullptr || (x.gather_rows > 0 && x.gather_rows < (1ll << 31) && x.gather_div > 0),
                "%s: gathered A needs 0 < rows < 2^31 and div > 0", name);
  MOE_CHECK_ARG(x.combine_row_src == nullptr || x.combine_topk > 0, "%s: topk must be positive", name);
  const moe_gemm_options o = resolve(options);
  GemmArgs args{};
  args.chunk_index = x.chunk_index;
  args.chunk_count = x.chunk_count;
  MOE_CHECK_ARG(o.expert_end <= o.expert_begin || (tile_pairs != nullptr && o.expert_begin >= 0 && o.expert_begin < E),
                "%s: the expert range [%d, %d) needs tile_pairs and 0 <= begin < num_experts", name, o.expert_begin,
                o.expert_end);
  args.expert_begin = o.expert_begin;
  args.expert_end = o.expert_end;
  MOE_CHECK_ARG(o.pair_end <= o.pair_begin || (tile_pairs != nullptr && o.pair_begin >= 0),
                "%s: the pair range [%d, %d) needs tile_pairs and begin >= 0", name, o.pair_begin, o.pair_end);
  args.pair_begin = o.pair_begin;
  args.pair_end = o.pair_end;
  args.mtile_expert = mtile_expert;
  args.tile_pairs = tile_pairs;
  args.mtiles_bound = static_cast<int32_t>(padded_rows / BM);
  args.pair_prefix = tile_pairs != nullptr ? tile_pairs + padded_rows / BM : nullptr;
  {
    // Expert-aligned groups pay off when an expert has enough row-tile pairs to fill a group by itself
    // (measured: -36 % DRAM reads, +4 % speed at 8 pairs per expert; slower at ~4 pairs per expert, where
    // groups spanning several experts keep more CTA pairs on the same row tiles).
    const long long mean_rows = (padded_rows - static_cast<long long>(E) * (BM - 1)) / E;
    args.align_experts = tile_pairs == nullptr ? 0 : (o.align_experts != 0 ? (o.align_experts > 0 ? 1 : 0)
                                                                          : (mean_rows >= 6 * 2 * BM ? 1 : 0));
  }
  args.num_mtiles = num_mtiles;
  args.num_experts = E;
  args.n_dim = N;
  args.k_dim = K;
  args.a_row_src = x.gather_row_src;
  args.a_div = x.gather_div;
  args.a_rows = static_cast<int32_t>(x.gather_rows);
  args.b_blocked = (!w_transposed && N % 64 == 0 && o.separate_copies == 0) ? 1 : 0;
  // plain stores in the padded layout leave through bulk tensor stores (64-column boxes: N a multiple of 64)
  args.out_tma = (epi == EPI_ACT && x.push_row == nullptr && x.combine_row_src == nullptr && out != nullptr && N % 64 == 0 &&
                  o.lane_stores == 0) ? 1 : 0;
  args.out = out;
  args.aux_out = x.aux_out;
  args.aux_in = x.aux_in;
  args.push_bases = x.push_bases;
  args.push_rank = x.push_rank;
  args.push_row = x.push_row;
  args.combine_row_src = x.combine_row_src;
  args.combine_scores = x.combine_scores;
  args.combine_topk = x.combine_topk;
  args.act = act;
  args.group_m = o.group_m > 0 ? o.group_m : kDefaultGroupM;
  args.wait_limit = wait_limit_cycles();
  args.status = status;
  LaunchParams lp;
  lp.stream = static_cast<cudaStream_t>(stream);
  lp.max_ctas = o.max_ctas > 0 ? o.max_ctas : 0;
  {
    // The wave barrier cuts the DRAM reads of every M-grouped GEMM to about the algorithmic bytes (gate/up at
    // the Mixtral shape: 6.4 -> 2.1 GB), but only long contractions get faster (K = 14336: -1.2 %, K = 28672:
    // -2 %); at K = 4096 the synchronised bursts on shared tiles cost more than the re-reads (+6 %).  Hence
    // on for K >= 8192 unless the caller says otherwise.
    const bool on = o.wave_sync != 0 ? o.wave_sync > 0 : K >= 8192;
    args.wave_counter = nullptr;
    args.wave_workers = o.wave_workers > 0 ? o.wave_workers : 0;  // 0: the launcher fills in its worker count
    if (on) {
      args.wave_counter = o.wave_counter;
      if (args.wave_counter == nullptr) {
        const int rc = ring_wave_counter(&args.wave_counter);
        if (rc != MOE_OK) return rc;
      }
      MOE_CUDA(cudaMemsetAsync(args.wave_counter, 0, sizeof(uint32_t), lp.stream));
    }
  }
  const int bn = pick_bn(N);
  // CTA pairs, unless the experts average at most one 128-row tile: a pair then has nothing for its second CTA, and
  // a work item streams half as many weight columns per tensor-core cycle as two independent CTAs do (measured at
  // 64 rows per expert, DeepSeek-V3 shape: gate/up 4.10 -> 2.69 ms, down 2.01 -> 1.38; at 16 rows per expert,
  // OLMoE shape: -6..12 %; at 128 rows per expert 0..5 %).
  const long long mean_rows_per_expert = (padded_rows - static_cast<long long>(E) * (BM - 1)) / E;
  const bool pairs = tile_pairs != nullptr && (o.single_cta == 0 ? mean_rows_per_expert > BM : o.single_cta < 0);
  const int64_t a_rows = x.gather_row_src != nullptr ? x.gather_rows : padded_rows;
#define MOE_MG(TYPE)                                                                                              \
  (pairs ? (bn == 256 ? mgrouped_dispatch<TYPE, 256, 2>(a, w, a_rows, K, N, E, w_transposed, epi, args, dtype, lp) \
                      : mgrouped_dispatch<TYPE, 128, 2>(a, w, a_rows, K, N, E, w_transposed, epi, args, dtype, lp)) \
         : (bn == 256 ? mgrouped_dispatch<TYPE, 256, 1>(a, w, a_rows, K, N, E, w_transposed, epi, args, dtype, lp) \
                      : mgrouped_dispatch<TYPE, 128, 1>(a, w, a_rows, K, N, E, w_transposed, epi, args, dtype, lp)))
  if (dtype == MOE_DTYPE_BF16) return MOE_MG(__nv_bfloat16);
  return MOE_MG(__half);
#undef MOE_MG
}

template <typename T, int BN, int CTAS>
static int kgrouped_dispatch(const void* a, const void* b, int64_t a_rows, int64_t padded_rows, int M, int N,
                             const GemmArgs& args, int dtype, const LaunchParams& lp) {
  CUtensorMap ta, tb;
  if (args.a_blocked) {
    int rc = make_tmap_blocked(&ta, dtype, a, (uint64_t)a_rows, (uint64_t)M, 0, BK, BM / 64);
    if (rc != MOE_OK) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)M, (uint64_t)a_rows};
    const uint32_t box[2] = {64, args.a_row_src != nullptr ? 1u : (uint32_t)BK};
    int rc = make_tmap(&ta, dtype, a, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  if (args.b_blocked) {
    int rc = make_tmap_blocked(&tb, dtype, b, (uint64_t)padded_rows, (uint64_t)N, 0, BK, (uint32_t)(BN / CTAS / 64));
    if (rc != MOE_OK) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)padded_rows};
    const uint32_t box[2] = {64, BK};
    int rc = make_tmap(&tb, dtype, b, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  CUtensorMap td = ta;
  if (args.out_tma) {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)args.num_experts};
    const uint32_t box[3] = {64, 32, 1};
    int rc = make_tmap(&td, dtype, args.out, 3, dims, box);
    if (rc != MOE_OK) return rc;
  }
  return args.a_row_src != nullptr ? launch<T, BN, false, false, EPI_ACT, true, CTAS, true>(ta, tb, ta, td, args, lp)
                                   : launch<T, BN, false, false, EPI_ACT, true, CTAS, false>(ta, tb, ta, td, args, lp);
}

static int kgrouped_common(const char* name, const void* a, int64_t gather_rows, const int32_t* gather_row_src,
                           int gather_div, const void* b, void* dw, const int32_t* pad_offsets, int64_t padded_rows, int M,
                           int N, int num_experts, int dtype, const moe_gemm_options* options, int32_t* status,
                           void* stream) {
  MOE_CHECK_ARG(a && b && dw && pad_offsets, "%s: null pointer argument", name);
  MOE_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(dw), "%s: pointers must be 16-byte aligned", name);
  MOE_CHECK_ARG(padded_rows > 0 && padded_rows % BM == 0, "%s: padded_rows=%lld must be a positive multiple of %d", name,
                (long long)padded_rows, BM);
  MOE_CHECK_ARG(M > 0 && N > 0 && num_experts > 0, "%s: M=%d N=%d E=%d must be positive", name, M, N, num_experts);
  if (M % 8 != 0 || N % 8 != 0) {
    set_error("%s: M=%d and N=%d must be multiples of 8", name, M, N);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(dtype == MOE_DTYPE_BF16 || dtype == MOE_DTYPE_F16, "%s: unknown dtype %d", name, dtype);
  MOE_CHECK_ARG(gather_row_src == nullptr || (gather_rows > 0 && gather_rows < (1ll << 31) && gather_div > 0),
                "%s: gathered A needs 0 < rows < 2^31 and div > 0", name);
  const moe_gemm_options o = resolve(options);
  GemmArgs args{};
  args.pad_offsets = pad_offsets;
  args.num_experts = num_experts;
  args.m_dim = M;
  args.n_dim = N;
  args.a_row_src = gather_row_src;
  args.a_div = gather_div;
  args.a_rows = static_cast<int32_t>(gather_rows);
  args.a_blocked = (gather_row_src == nullptr && M % 64 == 0 && o.separate_copies == 0) ? 1 : 0;
  args.b_blocked = (N % 64 == 0 && o.separate_copies == 0) ? 1 : 0;
  args.out_tma = (N % 64 == 0 && o.lane_stores == 0) ? 1 : 0;
  args.out = dw;
  args.act = MOE_ACT_NONE;
  args.group_m = o.group_m > 0 ? o.group_m : kDefaultGroupM;
  args.wait_limit = wait_limit_cycles();
  args.status = status;
  LaunchParams lp;
  lp.stream = static_cast<cudaStream_t>(stream);
  lp.max_ctas = o.max_ctas > 0 ? o.max_ctas : 0;
  const int bn = pick_bn(N);
  // CTA pairs unless the contraction is at most one 64-row step per expert on average (measured at 64 rows per
  // expert, DeepSeek-V3 shape: weight1 gradient 4.00 -> 3.48 ms; at 128 rows per expert pairs are 9 % faster)
  const long long mean_rows_per_expert = (padded_rows - static_cast<long long>(num_experts) * (BM - 1)) / num_experts;
  const bool pairs = o.single_cta == 0 ? mean_rows_per_expert > 64 : o.single_cta < 0;
  const int64_t a_rows = gather_row_src != nullptr ? gather_rows : padded_rows;
#define MOE_KG(TYPE)                                                                                      \
  (pairs ? (bn == 256 ? kgrouped_dispatch<TYPE, 256, 2>(a, b, a_rows, padded_rows, M, N, args, dtype, lp)  \
                      : kgrouped_dispatch<TYPE, 128, 2>(a, b, a_rows, padded_rows, M, N, args, dtype, lp)) \
         : (bn == 256 ? kgrouped_dispatch<TYPE, 256, 1>(a, b, a_rows, padded_rows, M, N, args, dtype, lp)  \
                      : kgrouped_dispatch<TYPE, 128, 1>(a, b, a_rows, padded_rows, M, N, args, dtype, lp)))
  if (dtype == MOE_DTYPE_BF16) return MOE_KG(__nv_bfloat16);
  return MOE_KG(__half);
#undef MOE_KG
}

static bool act_is_glu(int act) { return act == MOE_ACT_SWIGLU || act == MOE_ACT_GEGLU; }

}  // namespace moe

using namespace moe;

extern "C" int moe_mgrouped_gemm(const void* a, const void* w, void* out, void* pre_act, const int32_t* mtile_expert,
                                 const int32_t* tile_pairs, const int32_t* num_mtiles, int64_t padded_rows, int K,
                                 int N, int num_experts, int w_transposed, int act, int dtype, int chunk_index,
                                 int chunk_count, const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_NONE && act <= MOE_ACT_GELU_TANH, "moe_mgrouped_gemm: unknown activation %d", act);
  const bool glu = act_is_glu(act);
  MOE_CHECK_ARG(!(glu && w_transposed), "moe_mgrouped_gemm: gated activations need w as [E, K, N]");
  if (!glu && (act == MOE_ACT_NONE || pre_act == nullptr)) pre_act = nullptr;  // nothing to save without an activation
  MExtras x;
  x.aux_out = pre_act;
  x.chunk_index = chunk_index;
  x.chunk_count = chunk_count;
  const int epi = glu ? EPI_GLU : (pre_act != nullptr ? EPI_ACT_AUX : EPI_ACT);
  return mgrouped_common("moe_mgrouped_gemm", a, w, out, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K, N,
                         num_experts, w_transposed, epi, act, dtype, options, status, stream);
}

extern "C" int moe_mgrouped_gemm_gather(const void* src, int64_t src_rows, const int32_t* row_src, int div, const void* w,
                                        void* out, void* pre_act, const int32_t* mtile_expert, const int32_t* tile_pairs,
                                        const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                        int act, int dtype, const moe_gemm_options* options, int32_t* status,
                                        void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_NONE && act <= MOE_ACT_GELU_TANH, "moe_mgrouped_gemm_gather: unknown activation %d", act);
  MOE_CHECK_ARG(row_src != nullptr, "moe_mgrouped_gemm_gather: row_src is null");
  const bool glu = act_is_glu(act);
  if (!glu && (act == MOE_ACT_NONE || pre_act == nullptr)) pre_act = nullptr;
  MExtras x;
  x.aux_out = pre_act;
  x.gather_row_src = row_src;
  x.gather_div = div;
  x.gather_rows = src_rows;
  const int epi = glu ? EPI_GLU : (pre_act != nullptr ? EPI_ACT_AUX : EPI_ACT);
  return mgrouped_common("moe_mgrouped_gemm_gather", src, w, out, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K,
                         N, num_experts, 0, epi, act, dtype, options, status, stream);
}

extern "C" int moe_mgrouped_gemm_combine(const void* a, const void* w, void* out, const int32_t* row_src,
                                         const void* scores, int topk, const int32_t* mtile_expert,
                                         const int32_t* tile_pairs, const int32_t* num_mtiles, int64_t padded_rows, int K,
                                         int N, int num_experts, int w_transposed, int dtype,
                                         const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(row_src != nullptr && out != nullptr, "moe_mgrouped_gemm_combine: null pointer argument");
  MExtras x;
  x.combine_row_src = row_src;
  x.combine_scores = scores;
  x.combine_topk = topk;
  return mgrouped_common("moe_mgrouped_gemm_combine", a, w, out, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K,
                         N, num_experts, w_transposed, EPI_ACT, MOE_ACT_NONE, dtype, options, status, stream);
}

extern "C" int moe_mgrouped_gemm_dglu(const void* g, const void* w, const void* pre_act, void* d_pre,
                                      const int32_t* mtile_expert, const int32_t* tile_pairs,
                                      const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                      int act, int dtype, int chunk_index, int chunk_count,
                                      const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_SILU && act <= MOE_ACT_GELU_TANH, "moe_mgrouped_gemm_dglu: activation %d has no derivative here",
                act);
  MOE_CHECK_ARG(pre_act != nullptr, "moe_mgrouped_gemm_dglu: pre_act is null");
  MExtras x;
  x.aux_in = pre_act;
  x.chunk_index = chunk_index;
  x.chunk_count = chunk_count;
  return mgrouped_common("moe_mgrouped_gemm_dglu", g, w, d_pre, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K, N,
                         num_experts, 1, act_is_glu(act) ? EPI_DGLU : EPI_ACT_AUX, act, dtype, options, status, stream);
}

extern "C" int moe_mgrouped_gemm_push(const void* a, const void* w, void* const* peer_bases, const int32_t* dest_rank,
                                      const int32_t* dest_row, const int32_t* mtile_expert, const int32_t* tile_pairs,
                                      const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                      int w_transposed, int dtype, int chunk_index, int chunk_count,
                                      const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(peer_bases && dest_rank && dest_row, "moe_mgrouped_gemm_push: null pointer argument");
  MExtras x;
  x.push_bases = peer_bases;
  x.push_rank = dest_rank;
  x.push_row = dest_row;
  x.chunk_index = chunk_index;
  x.chunk_count = chunk_count;
  return mgrouped_common("moe_mgrouped_gemm_push", a, w, nullptr, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K,
                         N, num_experts, w_transposed, EPI_ACT, MOE_ACT_NONE, dtype, options, status, stream);
}

extern "C" int moe_mgrouped_gemm_scatter(const void* a, int64_t a_rows, const int32_t* a_row_src, int a_div,
                                         const void* w, void* out, const int32_t* out_rows, const int32_t* mtile_expert,
                                         const int32_t* tile_pairs, const int32_t* num_mtiles, int64_t padded_rows, int K,
                                         int N, int num_experts, int w_transposed, int act, int dtype,
                                         const moe_gemm_options* options, int32_t* status, void* stream) {
  MOE_CHECK_ARG(out != nullptr && out_rows != nullptr, "moe_mgrouped_gemm_scatter: null pointer argument");
  MOE_CHECK_ARG(act == MOE_ACT_NONE || act == MOE_ACT_SILU || act == MOE_ACT_GELU || act == MOE_ACT_GELU_TANH,
                "moe_mgrouped_gemm_scatter: activation %d is not an element-wise one", act);
  MExtras x;
  x.push_row = out_rows;
  if (a_row_src != nullptr) {
    x.gather_row_src = a_row_src;
    x.gather_div = a_div;
    x.gather_rows = a_rows;
  }
  return mgrouped_common("moe_mgrouped_gemm_scatter", a, w, out, x, mtile_expert, tile_pairs, num_mtiles, padded_rows, K,
                         N, num_experts, w_transposed, EPI_ACT, act, dtype, options, status, stream);
}

extern "C" int moe_kgrouped_gemm(const void* a, const void* b, void* dw, const int32_t* pad_offsets,
                                 int64_t padded_rows, int M, int N, int num_experts, int dtype,
                                 const moe_gemm_options* options, int32_t* status, void* stream) {
  return kgrouped_common("moe_kgrouped_gemm", a, 0, nullptr, 1, b, dw, pad_offsets, padded_rows, M, N, num_experts, dtype,
                         options, status, stream);
}

extern "C" int moe_kgrouped_gemm_gather(const void* src, int64_t src_rows, const int32_t* row_src, int div, const void* b,
                                        void* dw, const int32_t* pad_offsets, int64_t padded_rows, int M, int N,
                                        int num_experts, int dtype, const moe_gemm_options* options, int32_t* status,
                                        void* stream) {
  MOE_CHECK_ARG(row_src != nullptr, "moe_kgrouped_gemm_gather: row_src is null");
  return kgrouped_common("moe_kgrouped_gemm_gather", src, src_rows, row_src, div, b, dw, pad_offsets, padded_rows, M, N,
                         num_experts, dtype, options, status, stream);
}

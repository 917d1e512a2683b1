// The grouped-GEMM kernel of the MoE expert path on B200 tensor cores, and its launcher.
//
// One persistent, warp-specialised kernel template covers every contraction of the layer:
//
//   M-grouped (ragged rows, one weight matrix per expert), padded expert-sorted layout:
//     gate/up  : H = Xs @ W1[e]            A K-major, B MN-major ([E,K,N], N contiguous)
//     down     : Y = Act @ W2[e]           A K-major, B MN-major
//     dAct     : dA = Gs @ W2[e]^T         A K-major, B K-major  ([E,N,K], K contiguous)
//     dX       : dXs = dH @ W1[e]^T        A K-major, B K-major
//   K-grouped (contraction over an expert's rows, one output matrix per expert):
//     dW1[e] = Xs_e^T @ dH_e, dW2[e] = Act_e^T @ Gs_e      A and B both MN-major
//
// Roles inside a CTA (320 threads, one CTA per SM):
//   warp 0      : TMA producer  -- cp.async.bulk.tensor tile loads into a ring of shared-memory
//                 stages (128-byte swizzle), signalled by mbarriers.  In the GATHER variants of the
//                 template (a row map `a_row_src` is given) the A rows are GATHERED by the loads themselves:
//                 the 32 lanes issue one tile::gather4 copy each (4 rows x 128 bytes), so the token rows of
//                 an expert never have to be copied into the expert-sorted layout first.  A compile-time
//                 variant because this loop has no slack for branches it does not take;
//   warp 1      : MMA issuer    -- tcgen05.mma (128 x BN x 16 per CTA, fp32 accumulators in TMEM,
//                 two accumulator stages) and tcgen05.commit;
//                 both warps walk their loops with all 32 lanes (uniform control flow) and let one
//                 ELECTED lane issue; each probes the next stage's barrier one stage ahead.  (Issuing
//                 from a single lane inside a divergent branch cost ~100 cycles per tcgen05 instruction
//                 and left the tensor pipe idle 15 % of the time.)
//   warps 2..9  : epilogue      -- tcgen05.ld the accumulator (each warp its 32-lane quadrant and
//                 half of the columns), apply the fused epilogue and store through a swizzled
//                 shared-memory tile per warp, so that every global store covers whole row segments,
//                 locally or into another GPU's buffer.  The dGLU epilogue moves its rows with TMA:
//                 the saved product arrives by cp.async.bulk.tensor loads into the warp's staging tile
//                 (one chunk ahead) and the result leaves by a bulk tensor store from the same tile.
// The accumulator of tile i+1 is produced while tile i is being drained.
//
// CTA pairs (template parameter CTAS = 2, launched as clusters of two): the two CTAs of a pair work
// on two row tiles of the same expert against the same weight tile.  Each CTA loads its own 128 A
// rows and HALF of the B columns; one tcgen05.mma.cta_group::2 issued by the pair's leader spans
// both SMs (256 x BN accumulator, 128 rows in each CTA's TMEM) and reads the B halves from both
// CTAs' shared memory.  That halves the B bytes each SM pulls from L2 and reads from shared memory
// per FLOP.  Every CTA fetches its own tiles with its own loads; nothing is broadcast.  Operand
// arrival is credited to the leader's mbarriers, stage release and accumulator-ready signals go to
// both CTAs (one tcgen05.commit whose arrival is broadcast to the pair), accumulator-drained arrivals
// come back to the leader.
//
// Replaces the Triton kernels m_grouped_gemm_persistent_kernel / m_grouped_gemm_inner_kernel
// (reference: src/moe_explore/triton_kernels/m_grouped_gemm.py:33-267) and their epilogues
// (epilogue_split.py:4-44, triton_kernels/activation.py:5-45).
#pragma once

#include "common.cuh"

#include <atomic>

namespace moe {

constexpr int BM = 128;       // accumulator rows per CTA (= TMEM lanes)
constexpr int BK = 64;        // K extent of one shared-memory stage: 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;    // K extent of one tcgen05.mma for 16-bit inputs
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kWaveLead = 8;   // stages before the end of an item at which a worker announces the next wave
constexpr int kDefaultGroupM = 12;  // consecutive row units that share a sweep over column tiles (L2 reuse)
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaveWaitLimitCycles = 1ll << 21;  // ~1 ms: the wave barrier is an optimisation, not a dependency

// EPI_ACT_AUX is EPI_ACT plus either a second output (aux_out: the un-activated product, saved for backward)
// or a second input (aux_in: the saved product; the accumulator is multiplied by the activation's derivative
// there).  A separate instantiation, so that the plain-store kernels of the hot path carry none of it.
enum Epilogue : int { EPI_ACT = 0, EPI_GLU = 1, EPI_DGLU = 2, EPI_ACT_AUX = 3 };

struct GemmArgs {
  // scheduling
  const int32_t* mtile_expert;  // M-grouped: expert of each 128-row tile
  const int32_t* tile_pairs;    // M-grouped, CTA pairs: first tile | expert << 20 | (pair has a second tile) << 31
  const int32_t* pair_prefix;   // M-grouped: exclusive prefix of the per-expert pair counts [E+1]
  const int32_t* num_mtiles;    // M-grouped: device int32[4] = {tiles in use, tile pairs in use, tile bound, 0}
  const int32_t* pad_offsets;   // K-grouped: padded row offsets [E+1]
  int32_t mtiles_bound;         // M-grouped: padded_rows / 128 as the caller sees it (checked against num_mtiles[2])
  int32_t num_experts;
  int32_t m_dim;  // K-grouped: rows of each output matrix
  int32_t n_dim;  // accumulator columns (N of the contraction)
  int32_t k_dim;  // M-grouped: K of the contraction
  // MN-major operands whose contiguous extent is a multiple of 64 are described to the copy engine as
  // [blocks of 64][rows][64]: ONE copy per stage then fetches all the 64-element-wide column blocks of the tile
  // (one instruction instead of two to four; the blocks land exactly where separate copies put them).
  int32_t a_blocked;  // K-grouped A
  int32_t b_blocked;  // B, when it is MN-major
  // A rows gathered by the loads (null: A is stored in the padded layout).  Padded row p reads row
  // a_row_src[p] / a_div of the A tensor, zeros where a_row_src[p] < 0.  a_rows = rows of the A tensor.
  const int32_t* a_row_src;
  int32_t a_div;
  int32_t a_rows;
  // epilogue
  int32_t out_tma;     // EPI_ACT without a row map: tiles leave through bulk tensor stores (tmap_d covers `out`)
  void* out;           // EPI_ACT: [rows, N]; EPI_GLU: [rows, N/2]; EPI_DGLU: [rows, 2N]
  void* aux_out;       // EPI_GLU, EPI_ACT_AUX: un-activated product [rows, N] or null
  const void* aux_in;  // EPI_DGLU: saved un-activated product [rows, 2N]; EPI_ACT_AUX: the same, [rows, N], or null
  // EPI_ACT, M-grouped only: when push_row != null, accumulator row p is stored at row push_row[p] (skipped when
  // negative) instead of row p -- of `out`, or, when push_bases != null, of the [*, N] matrix based at
  // push_bases[push_rank[p]] (another GPU's buffer, peer-mapped; rows with push_rank[p] < 0 are not stored).
  void* const* push_bases;
  const int32_t* push_rank;
  const int32_t* push_row;
  // EPI_ACT, M-grouped only: when combine_row_src != null, accumulator row p is multiplied by
  // combine_scores[j] (j = combine_row_src[p], or by 1 when combine_scores is null) and ADDED to row j / combine_topk
  // of `out` with vector reductions; rows with j < 0 are skipped.  `out` must start at zero.
  const int32_t* combine_row_src;
  const void* combine_scores;
  int32_t combine_topk;
  int32_t act;
  int32_t chunk_index;  // M-grouped: process only the experts [E*index/count, E*(index+1)/count) (lets a caller
  int32_t chunk_count;  // pipeline row movement against the GEMM); count <= 1 = everything
  int32_t expert_begin;  // M-grouped: when expert_end > expert_begin, process exactly the experts [begin, end)
  int32_t expert_end;    // instead (slices of unequal size, e.g. chosen by row counts)
  int32_t pair_begin;    // M-grouped: when pair_end > pair_begin, process exactly the row-tile pairs [begin, end) of
  int32_t pair_end;      // the pair list instead (slices that may cut through an expert)
  int32_t align_experts;  // M-grouped CTA pairs: scheduling groups never span two experts
  uint32_t* wave_counter;  // non-null: workers start every work item together (grid-wide arrival counter, zeroed
                           // by the host before the launch)
  int32_t wave_workers;    // arrivals per wave the barrier waits for (the number of workers of the launch)
  int32_t group_m;  // row units per scheduling group
  long long wait_limit;  // cycles after which a device-side wait gives up
  int32_t* status;
};

struct TileCoord {
  int m0;       // first accumulator row of THIS CTA: padded row (M-grouped) or output-matrix row (K-grouped)
  int n0;       // first accumulator column of the tile
  int expert;
  int k_row0;   // K-grouped: first padded row of the contraction
  int kiters;   // number of BK-deep stages to contract
  bool active;  // false for the second CTA of a pair whose expert has an odd number of row tiles
};

// ----------------------------------------------------------------------------------
// Shared-memory matrix descriptors (64-bit) for tcgen05.mma.
//   bits  0-13  start address >> 4
//   bits 16-29  leading-dimension byte offset >> 4
//   bits 32-45  stride-dimension byte offset >> 4
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle mode (2 = 128-byte)
// K-major operand tile as TMA writes it with a {64 x rows} box: row r sits at r*128 bytes, 16-byte
// chunks XOR-swizzled by (r % 8); 8-row groups are 1024 bytes apart (stride offset); the
// leading offset is unused for swizzled K-major layouts.
// MN-major operand tile: each TMA box is {64 MN-elements x BK k-rows}: k-row at k*128 bytes;
// 8-k-row groups are 1024 bytes apart (stride offset); the next 64 MN-elements live in the
// next box, BK*128 bytes further (leading offset).
// ----------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor (32-bit): fp32 accumulate, 16-bit A/B format, operand majorness, N>>3, M>>4.
// With a CTA pair the instruction covers M = 256 rows (128 per CTA).
template <typename T, int BN, bool A_K, bool B_K, int CTAS>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  uint32_t d = 0;
  d |= 1u << 4;                       // D format: F32
  d |= Elem<T>::kUmmaFormat << 7;     // A format
  d |= Elem<T>::kUmmaFormat << 10;    // B format
  d |= (A_K ? 0u : 1u) << 15;         // A major: 0 = K, 1 = MN
  d |= (B_K ? 0u : 1u) << 16;         // B major
  d |= static_cast<uint32_t>(BN >> 3) << 17;
  d |= static_cast<uint32_t>((BM * CTAS) >> 4) << 24;
  return d;
}

// Shared-memory plan: [operand stages][epilogue staging][barriers].  The staging area holds, per epilogue warp,
// swizzled 32-row x 128-byte tiles: one for the plain-store and GLU epilogues, two for the dGLU epilogue (the
// saved product of the next chunk lands in one while the other is computed on and stored from), which costs the
// dGLU kernels one operand stage.
template <int BN, int CTAS, int EPI>
struct SmemPlan {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBCols = BN / CTAS;        // B columns held by one CTA
  static constexpr int kBBytes = kBCols * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingTile = 32 * 128;
  static constexpr int kTilesPerWarp = EPI == EPI_DGLU ? 2 : 1;
  static constexpr int kStagingBytes = kEpilogueWarps * kTilesPerWarp * kStagingTile;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kBudget = 232448 - 1024 - kBarrierBytes - kStagingBytes;  // 227 KB minus alignment slack
  static constexpr int kStages = (kBudget / kStageBytes) > 8 ? 8 : (kBudget / kStageBytes);
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

// The slice of the work a launch covers.
struct Window {
  int m_begin;  // first row unit (pair or tile) of the window
  int e0, e1;   // experts of the window (M-grouped)
  int p_end;    // CTA pairs: one past the last pair of the window (a window may begin and end inside an expert)
};

// Number of (row unit, column tile) work items and the row-unit / column-tile counts.  A row unit is
// one 128-row tile (one CTA) or a pair of them (CTA pair).
template <bool KG, int CTAS>
__device__ __forceinline__ int total_tiles(const GemmArgs& args, int& mt, int& nt, Window& win, int BN) {
  nt = (args.n_dim + BN - 1) / BN;
  win.m_begin = 0;
  win.e0 = 0;
  win.e1 = args.num_experts;
  win.p_end = 0x7FFFFFFF;
  if (KG) {
    mt = (args.m_dim + BM * CTAS - 1) / (BM * CTAS);
    return args.num_experts * mt * nt;
  }
  mt = args.num_mtiles[CTAS - 1];
  if (args.pair_prefix != nullptr) {
    if (args.num_mtiles[2] != args.mtiles_bound) {
      // the pair prefix sits at tile_pairs[bound]: metadata built for another bound cannot be walked
      if (threadIdx.x == 0 && args.status != nullptr) atomicCAS(args.status, 0, DS_BAD_LAYOUT);
      mt = 0;
      return 0;
    }
    const int pairs = args.num_mtiles[1];
    int p0, p1;
    if (args.pair_end > args.pair_begin) {
      // an explicit range of the pair list; the experts it touches are found by the search in decode_tile
      p0 = args.pair_begin < pairs ? args.pair_begin : pairs;
      p1 = args.pair_end < pairs ? args.pair_end : pairs;
    } else {
      if (args.expert_end > args.expert_begin) {
        win.e0 = args.expert_begin;
        win.e1 = args.expert_end < args.num_experts ? args.expert_end : args.num_experts;
      } else if (args.chunk_count > 1) {
        win.e0 = static_cast<int>(static_cast<long long>(args.num_experts) * args.chunk_index / args.chunk_count);
        win.e1 = static_cast<int>(static_cast<long long>(args.num_experts) * (args.chunk_index + 1) / args.chunk_count);
      }
      p0 = args.pair_prefix[win.e0];
      p1 = args.pair_prefix[win.e1];
    }
    win.p_end = p1;
    if (CTAS == 2) {
      win.m_begin = p0;
      mt = p1 - p0;
    } else {  // one-CTA kernels: the same window expressed in tiles
      const int tiles = args.num_mtiles[0];
      win.m_begin = p0 < pairs ? (args.tile_pairs[p0] & 0xFFFFF) : tiles;
      mt = (p1 < pairs ? (args.tile_pairs[p1] & 0xFFFFF) : tiles) - win.m_begin;
    }
  }
  return mt * nt;
}

// Order of the work items.  CTA pairs (M-grouped): expert by expert; inside an expert its pairs are walked in
// groups of `group_m`, and inside a group every column tile is visited for all pairs of the group before moving
// on.  The CTA pairs running at one time then share ONE expert's weight tiles and a small set of row tiles, which
// keeps both in L2 (groups that straddle experts doubled the weight tiles in flight and cost 1.5x the DRAM reads).
// One-CTA kernels and the K-grouped kernels use the same grouped walk without the expert alignment.
template <bool KG, int CTAS>
__device__ __forceinline__ TileCoord decode_tile(int t, int mt, int nt, const Window& win, const GemmArgs& args, int BN,
                                                 int rank) {
  TileCoord c;
  int expert = 0;
  int span = mt;       // row units the grouped walk below runs over
  int span_begin = win.m_begin;
  if (KG) {
    expert = t / (mt * nt);
    t -= expert * (mt * nt);
  } else if (CTAS == 2 && args.align_experts != 0) {
    // binary search: the expert whose pairs contain work item t
    const int base = win.m_begin;
    int lo = win.e0, hi = win.e1;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((__ldg(args.pair_prefix + mid) - base) * nt <= t) lo = mid; else hi = mid;
    }
    span_begin = __ldg(args.pair_prefix + lo);
    int span_end = __ldg(args.pair_prefix + lo + 1);
    // a window given as a pair range may begin or end inside this expert: walk only its part of the expert
    if (span_begin < base) span_begin = base;
    if (span_end > win.p_end) span_end = win.p_end;
    span = span_end - span_begin;
    t -= (span_begin - base) * nt;
  }
  // split the span into equal groups of at most args.group_m row units
  const int num_groups = (span + args.group_m - 1) / args.group_m;
  const int group_m = num_groups > 0 ? (span + num_groups - 1) / num_groups : 1;
  const int per_group = group_m * nt;
  const int g = t / per_group;
  const int rem = t - g * per_group;
  const int m_first = g * group_m;
  const int gm = min(group_m, span - m_first);
  const int n_idx = rem / gm;
  const int m_idx = span_begin + m_first + (rem - n_idx * gm);
  c.n0 = n_idx * BN;
  c.active = true;
  if (KG) {
    c.m0 = (m_idx * CTAS + rank) * BM;
    c.expert = expert;
    c.k_row0 = __ldg(args.pad_offsets + expert);
    c.kiters = (__ldg(args.pad_offsets + expert + 1) - c.k_row0) / BK;  // padded ranges are multiples of 128
  } else {
    int tile = m_idx;
    if (CTAS == 2) {
      // one load: first tile (bits 0-19), expert (bits 20-30), "has a second tile" (bit 31)
      const uint32_t info = static_cast<uint32_t>(__ldg(args.tile_pairs + m_idx));
      const bool second = (info >> 31) != 0;
      tile = static_cast<int>(info & 0xFFFFFu);
      c.expert = static_cast<int>((info >> 20) & 0x7FFu);
      c.active = rank == 0 || second;
      if (rank == 1 && second) tile += 1;  // an inactive second CTA re-reads the first tile and stores nothing
    } else {
      c.expert = __ldg(args.mtile_expert + tile);
    }
    c.m0 = tile * BM;
    c.k_row0 = 0;
    c.kiters = (args.k_dim + BK - 1) / BK;
  }
  return c;
}

// Wave barrier of the persistent workers.  With a static stride every worker's i-th work item belongs to the same
// "wave" of neighbouring tiles; workers that share operand tiles only hit in L2 while they stream through them
// together, and they drift apart after a few tiles (measured: DRAM reads of a long-K GEMM equal the algorithmic
// bytes for one wave, 1.4x for two, 3.9x for eight).  The leader's producer thread of every worker therefore
// arrives on a global counter a few stages BEFORE it finishes the items of wave i-1 and waits at the start
// of wave i until all workers have arrived: split like this the wait is short and the operand pipeline does not
// drain, while workers still stay within a few stages of each other.
//
// The barrier is only an optimisation, and it presumes that all workers are resident at the same time, which
// nothing guarantees when another kernel holds SMs.  So the wait is short (~1 ms) and a worker whose wait runs
// out does NOT abort: it records DS_WAVE_FALLBACK, stops waiting for the rest of the launch (it keeps arriving,
// so that the others are not held up by it) and carries on with the static stride.  Returns false on that.
__device__ __forceinline__ bool wave_wait(uint32_t* counter, uint32_t target, const WaitCtx& w) {
  const long long t0 = clock64();
  // a quarter of the general limit at most: the other roles of the CTA wait (bounded by the general limit) for
  // what this producer will load only after it has given up here
  const long long limit = (w.limit >> 2) < kWaveWaitLimitCycles ? (w.limit >> 2) : kWaveWaitLimitCycles;
  int spins = 0;
  while (true) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen >= target) return true;
    if (((++spins) & 15) == 0) {
      if (*w.abort_flag) return false;
      if (clock64() - t0 > limit) {
        if (w.status != nullptr) atomicCAS(w.status, 0, DS_WAVE_FALLBACK);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// 8 consecutive output elements (16 bytes) from 8 fp32 values.
template <typename T>
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 r;
  r.x = Elem<T>::pack2(v[0], v[1]);
  r.y = Elem<T>::pack2(v[2], v[3]);
  r.z = Elem<T>::pack2(v[4], v[5]);
  r.w = Elem<T>::pack2(v[6], v[7]);
  return r;
}

__device__ __forceinline__ float act_plain(float x, int act) {
  return act == MOE_ACT_SILU ? silu_f(x) : (act == MOE_ACT_GELU ? gelu_f(x) : gelu_tanh_f(x));
}
__device__ __forceinline__ float dact_plain(float x, int act) {
  return act == MOE_ACT_SILU ? dsilu_f(x) : (act == MOE_ACT_GELU ? dgelu_f(x) : dgelu_tanh_f(x));
}

// Source rows of four consecutive padded rows, as the gather4 copy wants them: row_src / div, or `oob` (a row
// index outside the tensor, which the copy fills with zeros) for padding rows.
__device__ __forceinline__ int4 gather_rows4(const int32_t* row_src, int first, int div, int oob) {
  const int4 j = __ldg(reinterpret_cast<const int4*>(row_src + first));
  int4 r;
  r.x = j.x < 0 ? oob : j.x / div;
  r.y = j.y < 0 ? oob : j.y / div;
  r.z = j.z < 0 ? oob : j.z / div;
  r.w = j.w < 0 ? oob : j.w / div;
  return r;
}

// tmap_a / tmap_b: the operands.  tmap_c / tmap_d (EPI_DGLU): the saved product and the output, both
// [rows, 2N] with a {64 columns, 32 rows} box.  tmap_d (EPI_ACT with out_tma): the output, [rows, N] or
// [E, M, N], same box.
template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG, int CTAS, bool GATHER>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_d,
                    const GemmArgs args) {
  using Plan = SmemPlan<BN, CTAS, EPI>;
  constexpr int kStages = Plan::kStages;
  constexpr bool kPair = CTAS == 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;  // 128-byte swizzle atoms need 1024-byte alignment
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  const uint32_t staging_addr = tiles_addr + kStages * Plan::kStageBytes;  // 1024-byte aligned as well
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Plan::kStageBytes + Plan::kStagingBytes);
  const uint32_t full_bar = smem_u32(bars);                     // [kStages]  (used in the leader CTA)
  const uint32_t empty_bar = smem_u32(bars + kStages);          // [kStages]  (one set per CTA)
  const uint32_t tfull_bar = smem_u32(bars + 2 * kStages);      // [2]        (one set per CTA)
  const uint32_t tempty_bar = smem_u32(bars + 2 * kStages + 2); // [2]        (used in the leader CTA)
  const uint32_t epi_bar = smem_u32(bars + 2 * kStages + 4);    // [kEpilogueWarps][2]  (dGLU side-input tiles)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + 2 * kEpilogueWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * 8 + 4 + 2 * kEpilogueWarps) * 8 + 8 <= Plan::kBarrierBytes, "barrier area too small");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = kPair ? static_cast<int>(cluster_ctarank()) : 0;  // 0 = leader of the pair
  const int unit = blockIdx.x / CTAS;        // persistent worker index (CTA or CTA pair)
  const int num_units = gridDim.x / CTAS;

  WaitCtx wctx;
  wctx.abort_flag = abort_flag;
  wctx.peer_abort = kPair ? mapa_shared(smem_u32(const_cast<int*>(abort_flag)), static_cast<uint32_t>(rank ^ 1)) : 0u;
  wctx.status = args.status;
  wctx.limit = args.wait_limit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + 8 * s, CTAS);   // one arrive.expect_tx per CTA
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, kEpilogueWarps * CTAS);
    }
    for (int i = 0; i < 2 * kEpilogueWarps; ++i) mbar_init(epi_bar + 8 * i, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (EPI == EPI_DGLU) tma_prefetch_desc(&tmap_c);
    if (EPI == EPI_DGLU || (EPI == EPI_ACT && args.out_tma)) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) {
    if (kPair) {
      tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();  // the peer's barriers must be initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int mt, nt;
  Window win;
  const int ntiles = total_tiles<KG, CTAS>(args, mt, nt, win, BN);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp walks the loop (uniform control flow); one elected lane issues the tile copies, and with
    // gathered A rows every lane issues one gather4 copy.
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool freed = false;  // the stage about to be filled was already seen free (probed one stage ahead)
      const int bcol = rank * Plan::kBCols;  // this CTA's share of the tile's B columns
      const uint64_t pol = l2_policy_evict_normal();
      // Gathered A rows are a compile-time variant: the mere presence of the gather branches in this loop (taken or
      // not) cost every kernel 15-25 % (measured: gate/up 3.30 -> 3.00 ms, weight1 gradient 3.43 -> 2.75 ms at the
      // Mixtral shape with the branches compiled out), because the loop then no longer is the short elected-lane
      // sequence the operand pipeline needs once per 512 tensor-core cycles.
      constexpr bool gather = GATHER;
      TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
      // M-grouped gather: lane l owns rows 4l..4l+3 of the tile for all of its stages
      int4 rows_next = make_int4(0, 0, 0, 0);
      if (gather && !KG && unit < ntiles) rows_next = gather_rows4(args.a_row_src, c_next.m0 + 4 * lane, args.a_div, args.a_rows);
      bool wave_sync = !KG && args.wave_counter != nullptr && rank == 0;
      int wave = 0;
      for (int t = unit; t < ntiles && ok; t += num_units, ++wave) {
        const TileCoord c = c_next;
        const int4 rows_m = rows_next;
        // fetch the next work item's coordinates now; the loads complete while this tile streams
        if (t + num_units < ntiles) {
          c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
          if (gather && !KG) rows_next = gather_rows4(args.a_row_src, c_next.m0 + 4 * lane, args.a_div, args.a_rows);
        }
        if (wave_sync && wave > 0 &&
            !__all_sync(0xFFFFFFFFu, wave_wait(args.wave_counter, static_cast<uint32_t>(args.wave_workers) * wave, wctx))) {
          if (*abort_flag) {
            ok = false;
            break;
          }
          wave_sync = false;  // the barrier ran out: static stride from here on (arrivals below continue)
        }
        // this worker's arrival for the NEXT wave goes out kWaveLead stages before this item ends
        const bool arrive_here = !KG && args.wave_counter != nullptr && rank == 0;
        const int arrive_kb = c.kiters > kWaveLead ? c.kiters - kWaveLead : 0;
        // K-grouped gather: lane l owns k-rows 4(l % 16)..+3 of box l / 16; the indices change every stage and are
        // fetched one stage ahead
        int4 rows_k = make_int4(0, 0, 0, 0);
        if (gather && KG && c.kiters > 0) rows_k = gather_rows4(args.a_row_src, c.k_row0 + 4 * (lane & 15), args.a_div, args.a_rows);
        for (int kb = 0; kb < c.kiters; ++kb) {
          if (arrive_here && kb == arrive_kb && lane == 0) atomicAdd(args.wave_counter, 1u);
          int4 rows_k_next = rows_k;
          if (gather && KG && kb + 1 < c.kiters)
            rows_k_next = gather_rows4(args.a_row_src, c.k_row0 + (kb + 1) * BK + 4 * (lane & 15), args.a_div, args.a_rows);
          if (!freed && !__all_sync(0xFFFFFFFFu, mbar_wait(empty_bar + 8 * stage, phase ^ 1, wctx, DS_TIMEOUT_PRODUCER))) {
            ok = false;
            break;
          }
          {
            const int ns = stage + 1 == kStages ? 0 : stage + 1;
            freed = __all_sync(0xFFFFFFFFu, mbar_test_wait(empty_bar + 8 * ns, stage + 1 == kStages ? phase : phase ^ 1));
          }
          const uint32_t sa = tiles_addr + stage * Plan::kStageBytes;
          const uint32_t sb = sa + Plan::kABytes;
          // the second CTA of a pair credits the LEADER's barrier: the leader issues the MMA that reads both halves
          const bool remote = kPair && rank != 0;
          const uint32_t fb = remote ? mapa_shared(full_bar + 8 * stage, 0) : full_bar + 8 * stage;
          const bool leader_lane = elect_one();
          if (leader_lane) {
            if (remote) mbar_arrive_expect_tx_cluster(fb, Plan::kStageBytes);
            else mbar_arrive_expect_tx(fb, Plan::kStageBytes);
          }
          if (gather) {
            // all 32 lanes: 4 rows x 128 bytes each = the whole 128 x 64 (or 64 x 128) A tile of the stage
            if (KG) {
              const uint32_t dst = sa + (lane >> 4) * (BK * 128) + (lane & 15) * 512;
              if (remote) tma_gather4_pair(dst, &tmap_a, c.m0 + 64 * (lane >> 4), rows_k, fb, pol);
              else tma_gather4(dst, &tmap_a, c.m0 + 64 * (lane >> 4), rows_k, fb, pol);
            } else {
              const uint32_t dst = sa + lane * 512;
              if (remote) tma_gather4_pair(dst, &tmap_a, kb * BK, rows_m, fb, pol);
              else tma_gather4(dst, &tmap_a, kb * BK, rows_m, fb, pol);
            }
          }
          if (!leader_lane) {
            // the other lanes only keep step
          } else if (remote) {
            if (KG) {
              const int krow = c.k_row0 + kb * BK;
              if (gather) {
              } else if (args.a_blocked) {
                tma_load_3d_pair(sa, &tmap_a, 0, krow, c.m0 >> 6, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmap_a, c.m0 + 64 * j, krow, fb, pol);
              }
              if (args.b_blocked) {
                tma_load_3d_pair(sb, &tmap_b, 0, krow, (c.n0 + bcol) >> 6, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, krow, fb, pol);
              }
            } else {
              if (!gather) tma_load_2d_pair(sa, &tmap_a, kb * BK, c.m0, fb, pol);
              if (B_K) {
                tma_load_3d_pair(sb, &tmap_b, kb * BK, c.n0 + bcol, c.expert, fb, pol);
              } else if (args.b_blocked) {
                tma_load_4d_pair(sb, &tmap_b, 0, kb * BK, (c.n0 + bcol) >> 6, c.expert, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_3d_pair(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, kb * BK, c.expert, fb, pol);
              }
            }
          } else {
            // single CTA, or the leader of a pair: everything is local
            if (KG) {
              const int krow = c.k_row0 + kb * BK;
              if (gather) {
              } else if (args.a_blocked) {
                tma_load_3d(sa, &tmap_a, 0, krow, c.m0 >> 6, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmap_a, c.m0 + 64 * j, krow, fb, pol);
              }
              if (args.b_blocked) {
                tma_load_3d(sb, &tmap_b, 0, krow, (c.n0 + bcol) >> 6, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_2d(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, krow, fb, pol);
              }
            } else {
              if (!gather) tma_load_2d(sa, &tmap_a, kb * BK, c.m0, fb, pol);
              if (B_K) {
                tma_load_3d(sb, &tmap_b, kb * BK, c.n0 + bcol, c.expert, fb, pol);
              } else if (args.b_blocked) {
                tma_load_4d(sb, &tmap_b, 0, kb * BK, (c.n0 + bcol) >> 6, c.expert, fb, pol);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_3d(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, kb * BK, c.expert, fb, pol);
              }
            }
          }
          __syncwarp();
          rows_k = rows_k_next;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!KG && args.wave_counter != nullptr && rank == 0 && lane == 0) {
        // workers without an item in the remaining waves still count, so that the others do not wait for them
        // (arrivals for waves up to `wave` were made inside the items that preceded them)
        const int waves = (ntiles + num_units - 1) / num_units;
        for (int w = wave + 1; w < waves; ++w) atomicAdd(args.wave_counter, 1u);
      }
      if (!ok) {
        // Let copies that were already issued land before the CTA releases its shared memory.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------
    // The whole warp walks the tile / stage loop (uniform control flow and operands); one elected lane issues
    // the tensor-core instructions.
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc<T, BN, A_K, B_K, CTAS>();
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      bool ready = false;  // the stage about to be consumed was already seen full
      TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
      for (int t = unit; t < ntiles && ok; t += num_units) {
        const TileCoord c = c_next;
        if (t + num_units < ntiles) c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
        if (c.kiters == 0) continue;  // empty expert: the epilogue writes zeros on its own
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1, wctx, DS_TIMEOUT_MMA))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < c.kiters; ++kb) {
          // `ready` was probed one stage ahead (below), so that the barrier's round trip to shared memory
          // overlaps the issue of the previous stage's MMAs; only a stage that was not there yet is waited for.
          if (!ready && !__all_sync(0xFFFFFFFFu, mbar_wait(full_bar + 8 * stage, phase, wctx, DS_TIMEOUT_MMA))) {
            ok = false;
            break;
          }
          tc_fence_after();
          {
            const int ns = stage + 1 == kStages ? 0 : stage + 1;
            ready = __all_sync(0xFFFFFFFFu, mbar_test_wait(full_bar + 8 * ns, stage + 1 == kStages ? phase ^ 1 : phase));
          }
          const uint32_t sa = tiles_addr + stage * Plan::kStageBytes;
          const uint32_t sb = sa + Plan::kABytes;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // K-major: step 16 elements (32 bytes) along the swizzled 128-byte row.
              // MN-major: step 16 k-rows of 128 bytes.
              const uint64_t da = A_K ? make_desc(sa + k * (UMMA_K * 2), 16, 1024)
                                      : make_desc(sa + k * (UMMA_K * 128), BK * 128, 1024);
              const uint64_t db = B_K ? make_desc(sb + k * (UMMA_K * 2), 16, 1024)
                                      : make_desc(sb + k * (UMMA_K * 128), BK * 128, 1024);
              if (kPair) umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
              else umma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            // free the stage in every CTA whose shared memory these MMAs read (one broadcast arrival)
            if (kPair) umma_commit_pair_both(empty_bar + 8 * stage);
            else umma_commit(empty_bar + 8 * stage);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        // accumulator complete: tell the epilogue warps of every CTA holding a part of it
        if (elect_one()) {
          if (kPair) umma_commit_pair_both(tfull_bar + 8 * acc);
          else umma_commit(tfull_bar + 8 * acc);
        }
        __syncwarp();
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok || *abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // Warp w reads TMEM lane quadrant (w % 4); the two warps of a quadrant split the columns.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kChunksPerWarp = BN / 32 / 2;
    const int chunk_begin = half * kChunksPerWarp;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    T* out = reinterpret_cast<T*>(args.out);
    T* aux_out = reinterpret_cast<T*>(args.aux_out);
    const T* aux_in = reinterpret_cast<const T*>(args.aux_in);
    const int N = args.n_dim;
    const uint32_t tempty_leader = kPair ? mapa_shared(tempty_bar, 0) : tempty_bar;
    // this warp's staging tile(s): 32 rows x 128 bytes, 16-byte pieces XOR-swizzled by (row % 8), i.e. the layout
    // the 128-byte-swizzle tensor copies read and write
    const uint32_t stage_base = staging_addr + (warp - 2) * (Plan::kTilesPerWarp * Plan::kStagingTile);
    const uint32_t my_epi_bar = epi_bar + (warp - 2) * 16;
    uint32_t q = 0;  // dGLU: running count of side-input tiles this warp has received (buffer = q & 1)
    const int co_row = lane >> 3;  // coalesced access: row within a group of four
    const int co_ck = lane & 7;    // and 16-byte piece of the row's 128 bytes
    TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
    for (int t = unit; t < ntiles; t += num_units) {
      const TileCoord c = c_next;
      if (t + num_units < ntiles) c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
      const bool have_acc = c.kiters != 0;
      const int row = c.m0 + row_in_tile;
      bool row_ok = c.active;
      long long out_row;  // row index into the output matrix
      T* row_out = out;  // base of the matrix this lane's row is stored into
      float row_scale = 1.0f;
      if (KG) {
        row_ok = row_ok && row < args.m_dim;
        out_row = static_cast<long long>(c.expert) * args.m_dim + row;
      } else {
        out_row = row;
        if (EPI == EPI_ACT && args.push_row != nullptr) {
          int32_t r = -1;
          if (row_ok) {
            if (args.push_bases != nullptr) {
              const int32_t rk = __ldg(args.push_rank + row);
              if (rk >= 0) {
                row_out = reinterpret_cast<T*>(args.push_bases[rk]);
                r = __ldg(args.push_row + row);
              }
            } else {
              r = __ldg(args.push_row + row);
            }
          }
          row_ok = r >= 0;
          if (row_ok) out_row = r;
        } else if (EPI == EPI_ACT && args.combine_row_src != nullptr) {
          const int32_t j = row_ok ? __ldg(args.combine_row_src + row) : -1;
          row_ok = j >= 0;
          if (row_ok) {
            out_row = j / args.combine_topk;
            if (args.combine_scores != nullptr) row_scale = Elem<T>::to_float(reinterpret_cast<const T*>(args.combine_scores)[j]);
          }
        }
      }
      const long long warp_row0 = static_cast<long long>(c.m0) + quad * 32;
      if (EPI == EPI_DGLU) {
        // The saved product does not depend on the accumulator: request the first chunk's tile before waiting
        // for the MMAs.  The buffer it lands in was last read by the store issued two chunks ago.
        const int col0 = c.n0 + chunk_begin * 32;
        if (c.active && col0 < N && lane == 0) {
          bulk_wait_read_all();
          const uint32_t bar = my_epi_bar + 8 * (q & 1);
          mbar_arrive_expect_tx(bar, Plan::kStagingTile);
          tma_load_2d_plain(stage_base + (q & 1) * Plan::kStagingTile, &tmap_c, 2 * col0, static_cast<int>(warp_row0), bar);
        }
        __syncwarp();
      }
      if (have_acc) {
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar + 8 * acc, acc_phase, wctx, DS_TIMEOUT_EPILOGUE))) break;
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (EPI == EPI_ACT || EPI == EPI_ACT_AUX) {
        // Plain store (optionally with an activation, optionally into another GPU's buffer, optionally scaled and
        // added into token-order rows): two 32-column chunks at a time go through the swizzled shared-memory tile so
        // that every store instruction of the warp writes four 128-byte row segments instead of 32 scattered
        // 16-byte pieces.
        // EPI_ACT_AUX with aux_out: pass 0 stores the un-activated product there, pass 1 the activated one
        // into out.  EPI_ACT_AUX with aux_in: one pass, accumulator * act'(saved product).
        const unsigned long long my_base = reinterpret_cast<unsigned long long>(row_out + out_row * N);
        const bool two_outputs = EPI == EPI_ACT_AUX && aux_out != nullptr;
        const unsigned long long my_aux = two_outputs ? reinterpret_cast<unsigned long long>(aux_out + out_row * N) : 0ull;
        const int first_pass = two_outputs ? 0 : 1;
        const bool accumulate = EPI == EPI_ACT && !KG && args.combine_row_src != nullptr;
        // Without a row map the 32-row x 64-column piece this warp has staged leaves as ONE bulk tensor store (the copy
        // engine clips it at the edges of the matrix) instead of eight 16-byte stores per lane; the staging tile is
        // written again only after that store has read it.
        const bool tma_out = EPI == EPI_ACT && args.out_tma != 0;
        const bool tile_stored = KG ? (c.m0 + quad * 32 < args.m_dim) : c.active;
#pragma unroll 1
        for (int chunk = chunk_begin; chunk < chunk_begin + kChunksPerWarp; chunk += 2) {
#pragma unroll 1
          for (int pass = first_pass; pass < 2; ++pass) {
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
              float v[32];
              if (have_acc) {
                uint32_t raw[32];
                tmem_ld_32x32(taddr + (chunk + hc) * 32, raw);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.0f;
              }
              if (EPI == EPI_ACT_AUX && aux_in != nullptr) {
                const int col = c.n0 + (chunk + hc) * 32;
                const T* src = aux_in + out_row * N + col;
#pragma unroll
                for (int qq = 0; qq < 4; ++qq) {
                  const uint4 h = (row_ok && col + qq * 8 < N) ? __ldg(reinterpret_cast<const uint4*>(src + qq * 8))
                                                               : make_uint4(0, 0, 0, 0);
                  const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                  for (int p2 = 0; p2 < 4; ++p2) {
                    const float2 pre = Elem<T>::unpack2(hw[p2]);
                    v[qq * 8 + 2 * p2] *= dact_plain(pre.x, args.act);
                    v[qq * 8 + 2 * p2 + 1] *= dact_plain(pre.y, args.act);
                  }
                }
              } else if (pass == 1 && args.act != MOE_ACT_NONE) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = act_plain(v[i], args.act);
              }
              if (accumulate) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= row_scale;
              }
              if (tma_out && hc == 0) {
                if (lane == 0) bulk_wait_read_all();  // the previous round's store has read the staging tile
                __syncwarp();
              }
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint4 u = pack8<T>(v + qq * 8);
                const uint32_t addr = stage_base + lane * 128 + (((hc * 4 + qq) ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                             : "memory");
              }
            }
            const int col_pair0 = c.n0 + chunk * 32;  // first of the 64 columns staged
            if (tma_out) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && tile_stored && col_pair0 < N) {
                if (KG) tma_store_3d(&tmap_d, col_pair0, c.m0 + quad * 32, c.expert, stage_base);
                else tma_store_2d(&tmap_d, col_pair0, static_cast<int>(warp_row0), stage_base);
                bulk_commit();
              }
              continue;
            }
            __syncwarp();
            const unsigned long long pass_base = pass == 0 ? my_aux : my_base;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int r = j * 4 + co_row;  // row of the warp's 32 this lane writes in this step
              const unsigned long long base = __shfl_sync(0xFFFFFFFFu, pass_base, r);
              const int ok = __shfl_sync(0xFFFFFFFFu, row_ok ? 1 : 0, r);
              uint4 u;
              const uint32_t addr = stage_base + r * 128 + ((co_ck ^ (r & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
              const int col = col_pair0 + co_ck * 8;
              if (ok && col < N) {
                if (accumulate) red_add_v8<T>(reinterpret_cast<T*>(base) + col, u);
                else *reinterpret_cast<uint4*>(reinterpret_cast<T*>(base) + col) = u;
              }
            }
            __syncwarp();
          }  // pass
        }
      } else if (EPI == EPI_GLU) {
        // Two 32-column chunks per round.  The un-activated product (128 bytes per row) and the activated
        // half (64 bytes per row) each go through the warp's swizzled shared-memory tile, so that every store
        // instruction writes whole row segments (4 rows x 128 bytes, then 8 rows x 64 bytes) instead of 32
        // scattered 16-byte pieces.  Rows are valid or not per CTA here (no per-row mask).
        const int half_n = N >> 1;
#pragma unroll 1
        for (int chunk = chunk_begin; chunk < chunk_begin + kChunksPerWarp; chunk += 2) {
          uint4 act_pk[4];  // this lane's 32 activated values of the round
          const int col0 = c.n0 + chunk * 32;
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            float v[32];
            if (have_acc) {
              uint32_t raw[32];
              tmem_ld_32x32(taddr + (chunk + hc) * 32, raw);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0.0f;
            }
            if (aux_out != nullptr) {
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const uint4 u = pack8<T>(v + qq * 8);
                const uint32_t addr = stage_base + lane * 128 + (((hc * 4 + qq) ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                             : "memory");
              }
            }
            float g[16];
            if (args.act == MOE_ACT_GEGLU) {
#pragma unroll
              for (int i = 0; i < 16; ++i) g[i] = gelu_f(v[2 * i]) * v[2 * i + 1];
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) g[i] = silu_f(v[2 * i]) * v[2 * i + 1];
            }
            act_pk[hc * 2] = pack8<T>(g);
            act_pk[hc * 2 + 1] = pack8<T>(g + 8);
          }
          if (aux_out != nullptr) {
            __syncwarp();
            const bool ok = row_ok && col0 + co_ck * 8 < N;
            T* dst = aux_out + (warp_row0 + co_row) * N + col0 + co_ck * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int r = j * 4 + co_row;
              uint4 u;
              const uint32_t addr = stage_base + r * 128 + ((co_ck ^ (r & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
              if (ok) *reinterpret_cast<uint4*>(dst + static_cast<long long>(j) * 4 * N) = u;
            }
            __syncwarp();
          }
          // activated half: 4 pieces per row; slot = (piece | odd row << 2) ^ (row >> 1 & 3) keeps both the
          // row-per-lane writes and the 8-rows-per-instruction reads free of bank conflicts
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int slot = (i | ((lane & 1) << 2)) ^ ((lane >> 1) & 3);
            const uint32_t addr = stage_base + lane * 128 + (slot << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(act_pk[i].x), "r"(act_pk[i].y),
                         "r"(act_pk[i].z), "r"(act_pk[i].w)
                         : "memory");
          }
          __syncwarp();
          {
            const int hr = lane >> 2;  // row within a group of eight
            const int hk = lane & 3;   // 16-byte piece of the row's 64 bytes
            const int hcol = (col0 >> 1) + hk * 8;
            const bool ok = row_ok && hcol < half_n;
            T* dst = out + (warp_row0 + hr) * half_n + hcol;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int r = j * 8 + hr;
              const int slot = (hk | ((r & 1) << 2)) ^ ((r >> 1) & 3);
              uint4 u;
              const uint32_t addr = stage_base + r * 128 + (slot << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
              if (ok) *reinterpret_cast<uint4*>(dst + static_cast<long long>(j) * 8 * half_n) = u;
            }
          }
          __syncwarp();
        }
      } else {
        // EPI_DGLU: per 32 accumulator columns, 64 columns (128 bytes per row) of the saved product come in and as
        // many of the result go out, both as tensor copies of this warp's 32 x 128-byte tile; the lanes only read
        // their row from shared memory, do the math on the accumulator and write the row back in place.
        bool failed = false;
#pragma unroll 1
        for (int chunk = chunk_begin; chunk < chunk_begin + kChunksPerWarp; ++chunk) {
          const int col0 = c.n0 + chunk * 32;
          const bool live = c.active && col0 < N;  // uniform over the warp
          const uint32_t buf = stage_base + (q & 1) * Plan::kStagingTile;
          uint4 h_cur[8];
          if (live) {
            const int ncol0 = col0 + 32;
            if (chunk + 1 < chunk_begin + kChunksPerWarp && ncol0 < N && lane == 0) {
              // next chunk's tile into the other buffer, once the store that last read it is done with it
              bulk_wait_read_all();
              const uint32_t nbar = my_epi_bar + 8 * ((q + 1) & 1);
              mbar_arrive_expect_tx(nbar, Plan::kStagingTile);
              tma_load_2d_plain(stage_base + ((q + 1) & 1) * Plan::kStagingTile, &tmap_c, 2 * ncol0,
                                static_cast<int>(warp_row0), nbar);
            }
            __syncwarp();
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(my_epi_bar + 8 * (q & 1), (q >> 1) & 1, wctx, DS_TIMEOUT_EPILOGUE))) {
              failed = true;
              break;
            }
#pragma unroll
            for (int qq = 0; qq < 8; ++qq) {
              const uint32_t addr = buf + lane * 128 + ((qq ^ (lane & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(h_cur[qq].x), "=r"(h_cur[qq].y), "=r"(h_cur[qq].z), "=r"(h_cur[qq].w)
                           : "r"(addr));
            }
          }
          __syncwarp();  // tcgen05.ld is warp-collective
          float v[32];
          if (have_acc) {
            uint32_t raw[32];
            tmem_ld_32x32(taddr + chunk * 32, raw);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.0f;
          }
          if (live) {
            // v = d(activated)[row, col0..col0+32); pre-activation (gate, up) pairs at columns 2*col
#pragma unroll
            for (int qq = 0; qq < 8; ++qq) {  // 8 pre-activation elements = 4 (gate, up) pairs per 16 bytes
              const uint32_t hw[4] = {h_cur[qq].x, h_cur[qq].y, h_cur[qq].z, h_cur[qq].w};
              float o[8];
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                const float2 gu = Elem<T>::unpack2(hw[p]);
                const float da = v[qq * 4 + p];
                float act_g, dact_g;
                if (args.act == MOE_ACT_GEGLU) {
                  act_g = gelu_f(gu.x);
                  dact_g = dgelu_f(gu.x);
                } else {
                  const float sg = sigmoidf_fast(gu.x);
                  act_g = gu.x * sg;
                  dact_g = sg * (1.0f + gu.x * (1.0f - sg));
                }
                o[2 * p] = da * gu.y * dact_g;
                o[2 * p + 1] = da * act_g;
              }
              const uint4 u = pack8<T>(o);
              const uint32_t addr = buf + lane * 128 + ((qq ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                           : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_d, 2 * col0, static_cast<int>(warp_row0), buf);
              bulk_commit();
            }
            ++q;
          }
        }
        if (failed) break;
      }
      if (have_acc) {
        // this warp has read its part of the accumulator: one arrival per warp on the leader's barrier
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (kPair && rank != 0) mbar_arrive_cluster(tempty_leader + 8 * acc);
          else mbar_arrive(tempty_bar + 8 * acc);
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if ((EPI == EPI_DGLU || EPI == EPI_ACT) && lane == 0) bulk_wait_all();  // this warp's bulk stores are complete
  }

  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();  // neither CTA may exit while its peer can still touch its memory or barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ----------------------------------------------------------------------------------
// launcher (one explicit instantiation per kernel variant, spread over the gemm_inst_*.cu files)
// ----------------------------------------------------------------------------------
struct LaunchParams {
  int max_ctas;  // 0 = one CTA per SM
  cudaStream_t stream;
};

// Launches one kernel variant with as many persistent workers as fit the current device (capped by lp.max_ctas).
template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG, int CTAS, bool GATHER>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& td, GemmArgs args,
           const LaunchParams& lp);

#ifdef MOE_GEMM_DEFINE_LAUNCH
template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG, int CTAS, bool GATHER>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& td, GemmArgs args,
           const LaunchParams& lp) {
  auto kernel = grouped_gemm_kernel<T, BN, A_K, B_K, EPI, KG, CTAS, GATHER>;
  constexpr int smem = SmemPlan<BN, CTAS, EPI>::kTotal;
  static_assert(SmemPlan<BN, CTAS, EPI>::kStages >= 3, "too few operand stages");
  static std::atomic<int> grid_for_device[64];  // 0 = not configured yet (zero-initialised)
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = lp.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTAS > 1 ? 1 : 0;
  int grid = (dev >= 0 && dev < 64) ? grid_for_device[dev].load(std::memory_order_acquire) : 0;
  if (grid == 0) {
    // First launch of this variant on this device (two threads racing here compute the same value twice).
    MOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    grid = sm_count() / CTAS * CTAS;
    if (CTAS > 1) {
      // The tile loop is statically strided over the resident workers, so launch exactly as many
      // CTA pairs as can be resident at once (a GPC with an odd SM count cannot host a last pair).
      cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
      int clusters = 0;
      MOE_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
      if (clusters <= 0) {
        set_error("grouped GEMM: no CTA pair of this kernel fits on the device");
        return MOE_ERR_UNSUPPORTED;
      }
      if (clusters * CTAS < grid) grid = clusters * CTAS;
    }
    if (dev >= 0 && dev < 64) grid_for_device[dev].store(grid, std::memory_order_release);
  }
  {
    const int limit = lp.max_ctas / CTAS * CTAS;
    if (limit >= CTAS && limit < grid) grid = limit;
  }
  if (args.wave_workers <= 0) args.wave_workers = grid / CTAS;
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  MOE_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, td, args));
  return MOE_OK;
}
#endif  // MOE_GEMM_DEFINE_LAUNCH

}  // namespace moe

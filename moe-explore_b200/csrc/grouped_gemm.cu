// Grouped GEMMs for the MoE expert path on B200 tensor cores.
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
//                 stages (128-byte swizzle), signalled by mbarriers;
//   warp 1      : MMA issuer    -- tcgen05.mma (128 x BN x 16 per CTA, fp32 accumulators in TMEM,
//                 two accumulator stages) and tcgen05.commit;
//                 both warps walk their loops with all 32 lanes (uniform control flow) and let one
//                 ELECTED lane issue; each probes the next stage's barrier one stage ahead.  (Issuing
//                 from a single lane inside a divergent branch cost ~100 cycles per tcgen05 instruction
//                 and left the tensor pipe idle 15 % of the time.)
//   warps 2..9  : epilogue      -- tcgen05.ld the accumulator (each warp its 32-lane quadrant and
//                 half of the columns), apply the fused epilogue and store through a swizzled
//                 shared-memory tile per warp, so that every global store (and the dGLU loads) covers
//                 whole row segments, locally or into another GPU's buffer.
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
// (epilogue_split.py:4-44, triton_kernels/activation.py:5-36).
#include "common.cuh"

#include <stdlib.h>

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

// EPI_ACT_AUX is EPI_ACT plus either a second output (aux_out: the un-activated product, saved for backward)
// or a second input (aux_in: the saved product; the accumulator is multiplied by the activation's derivative
// there).  A separate instantiation, so that the plain-store kernels of the hot path carry none of it.
enum Epilogue : int { EPI_ACT = 0, EPI_GLU = 1, EPI_DGLU = 2, EPI_ACT_AUX = 3 };

struct GemmArgs {
  // scheduling
  const int32_t* mtile_expert;  // M-grouped: expert of each 128-row tile
  const int32_t* tile_pairs;    // M-grouped, CTA pairs: first tile | expert << 20 | (pair has a second tile) << 31
  const int32_t* pair_prefix;   // M-grouped: exclusive prefix of the per-expert pair counts [E+1]
  const int32_t* num_mtiles;    // M-grouped: device int32[2] = {tiles in use, tile pairs in use}
  const int32_t* pad_offsets;   // K-grouped: padded row offsets [E+1]
  int32_t num_experts;
  int32_t m_dim;  // K-grouped: rows of each output matrix
  int32_t n_dim;  // accumulator columns (N of the contraction)
  int32_t k_dim;  // M-grouped: K of the contraction
  // epilogue
  void* out;           // EPI_ACT: [rows, N]; EPI_GLU: [rows, N/2]; EPI_DGLU: [rows, 2N]
  void* aux_out;       // EPI_GLU, EPI_ACT_AUX: un-activated product [rows, N] or null
  const void* aux_in;  // EPI_DGLU: saved un-activated product [rows, 2N]; EPI_ACT_AUX: the same, [rows, N], or null
  // EPI_ACT, M-grouped only: when push_bases != null, accumulator row p is stored at row push_row[p] of the
  // [*, N] matrix based at push_bases[push_rank[p]] (another GPU's buffer, peer-mapped) instead of `out`;
  // rows with push_rank[p] < 0 are not stored.
  void* const* push_bases;
  const int32_t* push_rank;
  const int32_t* push_row;
  int32_t act;
  int32_t chunk_index;  // M-grouped: process only the experts [E*index/count, E*(index+1)/count) (lets a caller
  int32_t chunk_count;  // pipeline row movement against the GEMM); count <= 1 = everything
  int32_t align_experts;  // M-grouped CTA pairs: scheduling groups never span two experts
  uint32_t* wave_counter;  // non-null: workers start every wave_period-th work item together (grid-wide arrival
                           // counter, zeroed by the host before the launch)
  int32_t wave_period;
  int32_t group_m;  // row units per scheduling group
  int32_t hint_weights_stream;  // 1: weight tiles get the evict-first L2 policy
  int32_t* status;
#ifdef MOE_GEMM_STATS
  long long* stats;  // [grid][4]: MMA thread cycles {total, waiting for operands, waiting for a free accumulator, tiles}
#endif
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

template <int BN, int CTAS>
struct SmemPlan {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBCols = BN / CTAS;        // B columns held by one CTA
  static constexpr int kBBytes = kBCols * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  static constexpr int kBarrierBytes = 256;
  // plain-store epilogue: each epilogue warp stages 32 rows x 64 columns (128 bytes per row) so that
  // its global stores cover whole 128-byte row segments
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + kStagingBytes + 1024;  // + alignment slack
};

// The slice of the work a launch covers.
struct Window {
  int m_begin;  // first row unit (pair or tile) of the window
  int e0, e1;   // experts of the window (M-grouped)
};

// Number of (row unit, column tile) work items and the row-unit / column-tile counts.  A row unit is
// one 128-row tile (one CTA) or a pair of them (CTA pair).
template <bool KG, int CTAS>
__device__ __forceinline__ int total_tiles(const GemmArgs& args, int& mt, int& nt, Window& win, int BN) {
  nt = (args.n_dim + BN - 1) / BN;
  win.m_begin = 0;
  win.e0 = 0;
  win.e1 = args.num_experts;
  if (KG) {
    mt = (args.m_dim + BM * CTAS - 1) / (BM * CTAS);
    return args.num_experts * mt * nt;
  }
  mt = args.num_mtiles[CTAS - 1];
  if (args.pair_prefix != nullptr) {
    if (args.chunk_count > 1) {
      win.e0 = static_cast<int>(static_cast<long long>(args.num_experts) * args.chunk_index / args.chunk_count);
      win.e1 = static_cast<int>(static_cast<long long>(args.num_experts) * (args.chunk_index + 1) / args.chunk_count);
    }
    const int pairs = args.num_mtiles[1];
    const int p0 = args.pair_prefix[win.e0], p1 = args.pair_prefix[win.e1];
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
    span = __ldg(args.pair_prefix + lo + 1) - span_begin;
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
// arrives on a global counter a few stages BEFORE it finishes the items of wave i-1 and waits (bounded) at the start
// of wave i until all workers have arrived: split like this the wait is short and the operand pipeline does not
// drain, while workers still stay within a few stages of each other.
__device__ __forceinline__ bool wave_wait(uint32_t* counter, uint32_t target, volatile int* abort_flag, int* status) {
  const long long t0 = clock64();
  int spins = 0;
  while (true) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen >= target) return true;
    if (((++spins) & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, DS_TIMEOUT_PRODUCER);
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

template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs args) {
  using Plan = SmemPlan<BN, CTAS>;
  constexpr int kStages = Plan::kStages;
  constexpr bool kPair = CTAS == 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;  // 128-byte swizzle atoms need 1024-byte alignment
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Plan::kStageBytes);
  const uint32_t full_bar = smem_u32(bars);                     // [kStages]  (used in the leader CTA)
  const uint32_t empty_bar = smem_u32(bars + kStages);          // [kStages]  (one set per CTA)
  const uint32_t tfull_bar = smem_u32(bars + 2 * kStages);      // [2]        (one set per CTA)
  const uint32_t tempty_bar = smem_u32(bars + 2 * kStages + 2); // [2]        (used in the leader CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = kPair ? static_cast<int>(cluster_ctarank()) : 0;  // 0 = leader of the pair
  const int unit = blockIdx.x / CTAS;        // persistent worker index (CTA or CTA pair)
  const int num_units = gridDim.x / CTAS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + 8 * s, CTAS);   // one arrive.expect_tx per CTA
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, kEpilogueWarps * CTAS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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
    // The whole warp walks the loop (uniform control flow); one elected lane issues the copies.
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool freed = false;  // the stage about to be filled was already seen free (probed one stage ahead)
      const int bcol = rank * Plan::kBCols;  // this CTA's share of the tile's B columns
      // L2 eviction priority of the operand tiles.  Default: normal priority for both.  Measured on the
      // Mixtral shape, marking the row tiles evict-last and the weight tiles evict-first RAISED the DRAM
      // reads of the gate/up GEMM from 6.4 GB to 9.7 GB (weight tiles shared by the CTA pairs of one
      // expert were dropped before every pair had read them), so it is opt-in for experiments only.
      const bool hinted = !KG && args.hint_weights_stream != 0;
      const uint64_t pol_a = hinted ? l2_policy_evict_last() : l2_policy_evict_normal();
      const uint64_t pol_b = hinted ? l2_policy_evict_first() : l2_policy_evict_normal();
      TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
      const bool wave_sync = !KG && args.wave_counter != nullptr && rank == 0;
      int wave = 0;
      for (int t = unit; t < ntiles && ok; t += num_units, ++wave) {
        const TileCoord c = c_next;
        // fetch the next work item's coordinates now; the loads complete while this tile streams
        if (t + num_units < ntiles) c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
        if (wave_sync && wave > 0 && wave % args.wave_period == 0 &&
            !__all_sync(0xFFFFFFFFu, wave_wait(args.wave_counter, static_cast<uint32_t>(num_units) * (wave / args.wave_period),
                                               abort_flag, args.status))) {
          ok = false;
          break;
        }
        // this worker's arrival for the NEXT synchronised wave goes out kWaveLead stages before this item ends
        const bool arrive_here = wave_sync && (wave + 1) % args.wave_period == 0;
        const int arrive_kb = c.kiters > kWaveLead ? c.kiters - kWaveLead : 0;
        for (int kb = 0; kb < c.kiters; ++kb) {
          if (arrive_here && kb == arrive_kb && lane == 0) atomicAdd(args.wave_counter, 1u);
          if (!freed && !__all_sync(0xFFFFFFFFu, mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, args.status,
                                                           DS_TIMEOUT_PRODUCER))) {
            ok = false;
            break;
          }
          {
            const int ns = stage + 1 == kStages ? 0 : stage + 1;
            freed = __all_sync(0xFFFFFFFFu, mbar_test_wait(empty_bar + 8 * ns, stage + 1 == kStages ? phase : phase ^ 1));
          }
          const uint32_t sa = tiles_addr + stage * Plan::kStageBytes;
          const uint32_t sb = sa + Plan::kABytes;
          if (!elect_one()) {
            // the other lanes only keep step
          } else if (kPair && rank != 0) {
            // the second CTA credits the LEADER's barrier: the leader issues the MMA that reads both halves
            const uint32_t fb = mapa_shared(full_bar + 8 * stage, 0);
            mbar_arrive_expect_tx_cluster(fb, Plan::kStageBytes);
            if (KG) {
              const int krow = c.k_row0 + kb * BK;
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmap_a, c.m0 + 64 * j, krow, fb, pol_a);
#pragma unroll
              for (int j = 0; j < Plan::kBCols / 64; ++j)
                tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, krow, fb, pol_b);
            } else {
              tma_load_2d_pair(sa, &tmap_a, kb * BK, c.m0, fb, pol_a);
              if (B_K) {
                tma_load_3d_pair(sb, &tmap_b, kb * BK, c.n0 + bcol, c.expert, fb, pol_b);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_3d_pair(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, kb * BK, c.expert, fb, pol_b);
              }
            }
          } else {
            // single CTA, or the leader of a pair: everything is local
            const uint32_t fb = full_bar + 8 * stage;
            mbar_arrive_expect_tx(fb, Plan::kStageBytes);
            if (KG) {
              const int krow = c.k_row0 + kb * BK;
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmap_a, c.m0 + 64 * j, krow, fb, pol_a);
#pragma unroll
              for (int j = 0; j < Plan::kBCols / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, krow, fb, pol_b);
            } else {
              tma_load_2d(sa, &tmap_a, kb * BK, c.m0, fb, pol_a);
              if (B_K) {
                tma_load_3d(sb, &tmap_b, kb * BK, c.n0 + bcol, c.expert, fb, pol_b);
              } else {
#pragma unroll
                for (int j = 0; j < Plan::kBCols / 64; ++j)
                  tma_load_3d(sb + j * (BK * 128), &tmap_b, c.n0 + bcol + 64 * j, kb * BK, c.expert, fb, pol_b);
              }
            }
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (wave_sync && lane == 0) {
        // workers without an item in the remaining waves still count, so that the others do not wait for them
        // (arrivals for waves up to `wave` were made inside the items that preceded them)
        const int waves = (ntiles + num_units - 1) / num_units;
        for (int w = wave + 1; w < waves; ++w)
          if (w % args.wave_period == 0) atomicAdd(args.wave_counter, 1u);
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
#ifdef MOE_GEMM_STATS
      long long st_total = clock64(), st_full = 0, st_acc = 0, st_tiles = 0, st_slow_n = 0, st_slow = 0, st_issue = 0, st_stages = 0;
#endif
      TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
      for (int t = unit; t < ntiles && ok; t += num_units) {
        const TileCoord c = c_next;
        if (t + num_units < ntiles) c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
        if (c.kiters == 0) continue;  // empty expert: the epilogue writes zeros on its own
#ifdef MOE_GEMM_STATS
        const long long t_acc0 = clock64();
#endif
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, args.status, DS_TIMEOUT_MMA))) {
          ok = false;
          break;
        }
#ifdef MOE_GEMM_STATS
        st_acc += clock64() - t_acc0;
        ++st_tiles;
#endif
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < c.kiters; ++kb) {
#ifdef MOE_GEMM_STATS
          const long long t_full0 = clock64();
#endif
          // `ready` was probed one stage ahead (below), so that the barrier's round trip to shared memory
          // overlaps the issue of the previous stage's MMAs; only a stage that was not there yet is waited for.
          if (!ready && !__all_sync(0xFFFFFFFFu, mbar_wait(full_bar + 8 * stage, phase, abort_flag, args.status, DS_TIMEOUT_MMA))) {
            ok = false;
            break;
          }
#ifdef MOE_GEMM_STATS
          const long long t_full1 = clock64();
          st_full += t_full1 - t_full0;
          ++st_stages;
          if (t_full1 - t_full0 > 150) { ++st_slow_n; st_slow += t_full1 - t_full0; }
#endif
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
#ifdef MOE_GEMM_STATS
          st_issue += clock64() - t_full1;
#endif
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
#ifdef MOE_GEMM_STATS
      if (args.stats != nullptr && lane == 0) {
        long long* o = args.stats + 8 * blockIdx.x;
        o[0] = clock64() - st_total;
        o[1] = st_full;
        o[2] = st_acc;
        o[3] = st_tiles;
        o[4] = st_slow_n;
        o[5] = st_slow;
        o[6] = st_issue;
        o[7] = st_stages;
      }
#endif
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
    TileCoord c_next = decode_tile<KG, CTAS>(unit < ntiles ? unit : 0, mt, nt, win, args, BN, rank);
    for (int t = unit; t < ntiles; t += num_units) {
      const TileCoord c = c_next;
      if (t + num_units < ntiles) c_next = decode_tile<KG, CTAS>(t + num_units, mt, nt, win, args, BN, rank);
      const bool have_acc = c.kiters != 0;
      const int row = c.m0 + row_in_tile;
      bool row_ok = c.active;
      long long out_row;  // row index into the output matrix
      T* row_out = out;  // base of the matrix this lane's row is stored into
      if (KG) {
        row_ok = row_ok && row < args.m_dim;
        out_row = static_cast<long long>(c.expert) * args.m_dim + row;
      } else {
        out_row = row;
        if (EPI == EPI_ACT && args.push_bases != nullptr) {
          const int32_t r = row_ok ? __ldg(args.push_rank + row) : -1;
          row_ok = r >= 0;
          if (row_ok) {
            row_out = reinterpret_cast<T*>(args.push_bases[r]);
            out_row = __ldg(args.push_row + row);
          }
        }
      }
      // EPI_DGLU: the saved pre-activation does not depend on the accumulator -- fetch the first
      // chunk before waiting for the MMAs, then stay one chunk ahead.  Loads and stores are coalesced:
      // instruction j of a chunk covers rows 4j..4j+3 of the warp's 32, eight 16-byte pieces per row
      // (whole 128-byte lines); a swizzled 4 KB shared-memory tile per warp turns that into the
      // row-per-lane layout of the accumulator and back.  (One row per lane straight to global memory
      // cost 32 memory transactions per instruction and made short contractions epilogue-bound.)
      uint4 h_next[8];
      const long long ld2 = 2ll * N;
      const int co_row = lane >> 3;  // row within a group of four
      const int co_ck = lane & 7;    // 16-byte piece of the row's 128 bytes = 4 output columns
      const long long warp_row0 = static_cast<long long>(c.m0) + quad * 32;
      const uint32_t dglu_stage = tiles_addr + kStages * Plan::kStageBytes + Plan::kBarrierBytes + (warp - 2) * (32 * 128);
      if (EPI == EPI_DGLU) {
        const int col0 = c.n0 + chunk_begin * 32;
        const bool ok = row_ok && col0 + co_ck * 4 < N;
        const T* src = aux_in + (warp_row0 + co_row) * ld2 + 2 * col0 + co_ck * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          h_next[j] = ok ? __ldg(reinterpret_cast<const uint4*>(src + j * 4 * ld2)) : make_uint4(0, 0, 0, 0);
      }
      if (have_acc) {
        if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, args.status, DS_TIMEOUT_EPILOGUE)) break;
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (EPI == EPI_ACT || EPI == EPI_ACT_AUX) {
        // Plain store (optionally with silu/gelu, optionally into another GPU's buffer): two 32-column
        // chunks at a time go through a swizzled shared-memory tile so that every store instruction
        // of the warp writes four 128-byte row segments instead of 32 scattered 16-byte pieces.
        // EPI_ACT_AUX with aux_out: pass 0 stores the un-activated product there, pass 1 the activated one
        // into out.  EPI_ACT_AUX with aux_in: one pass, accumulator * act'(saved product).
        const uint32_t stage_base = tiles_addr + kStages * Plan::kStageBytes + Plan::kBarrierBytes + (warp - 2) * (32 * 128);
        const unsigned long long my_base = reinterpret_cast<unsigned long long>(row_out + out_row * N);
        const bool two_outputs = EPI == EPI_ACT_AUX && aux_out != nullptr;
        const unsigned long long my_aux = two_outputs ? reinterpret_cast<unsigned long long>(aux_out + out_row * N) : 0ull;
        const int first_pass = two_outputs ? 0 : 1;
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
              for (int q = 0; q < 4; ++q) {
                const uint4 h = (row_ok && col + q * 8 < N) ? __ldg(reinterpret_cast<const uint4*>(src + q * 8))
                                                            : make_uint4(0, 0, 0, 0);
                const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                for (int p2 = 0; p2 < 4; ++p2) {
                  const float2 pre = Elem<T>::unpack2(hw[p2]);
                  const bool gelu = args.act == MOE_ACT_GELU;
                  v[q * 8 + 2 * p2] *= gelu ? dgelu_f(pre.x) : dsilu_f(pre.x);
                  v[q * 8 + 2 * p2 + 1] *= gelu ? dgelu_f(pre.y) : dsilu_f(pre.y);
                }
              }
            } else if (pass == 1) {
              if (args.act == MOE_ACT_SILU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
              } else if (args.act == MOE_ACT_GELU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = gelu_f(v[i]);
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 u = pack8<T>(v + q * 8);
              const uint32_t addr = stage_base + lane * 128 + (((hc * 4 + q) ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                           : "memory");
            }
          }
          __syncwarp();
          const int col_pair0 = c.n0 + chunk * 32;  // first of the 64 columns staged
          const unsigned long long pass_base = pass == 0 ? my_aux : my_base;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = j * 4 + (lane >> 3);   // row of the warp's 32 this lane writes in this step
            const int ck = lane & 7;             // 16-byte piece of the row's 128 bytes
            const unsigned long long base = __shfl_sync(0xFFFFFFFFu, pass_base, r);
            const int ok = __shfl_sync(0xFFFFFFFFu, row_ok ? 1 : 0, r);
            uint4 u;
            const uint32_t addr = stage_base + r * 128 + ((ck ^ (r & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
            const int col = col_pair0 + ck * 8;
            if (ok && col < N) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(base) + col) = u;
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
              for (int q = 0; q < 4; ++q) {
                const uint4 u = pack8<T>(v + q * 8);
                const uint32_t addr = dglu_stage + lane * 128 + (((hc * 4 + q) ^ (lane & 7)) << 4);
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
              const uint32_t addr = dglu_stage + r * 128 + ((co_ck ^ (r & 7)) << 4);
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
            const uint32_t addr = dglu_stage + lane * 128 + (slot << 4);
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
              const uint32_t addr = dglu_stage + r * 128 + (slot << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
              if (ok) *reinterpret_cast<uint4*>(dst + static_cast<long long>(j) * 8 * half_n) = u;
            }
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int chunk = chunk_begin; chunk < chunk_begin + kChunksPerWarp; ++chunk) {
        float v[32];
        uint4 h_cur[8];
        const int col0 = c.n0 + chunk * 32;
        if (EPI == EPI_DGLU) {
          // this chunk's rows: coalesced registers -> shared memory -> one row per lane
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = j * 4 + co_row;
            const uint32_t addr = dglu_stage + r * 128 + ((co_ck ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(h_next[j].x), "r"(h_next[j].y),
                         "r"(h_next[j].z), "r"(h_next[j].w)
                         : "memory");
          }
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t addr = dglu_stage + lane * 128 + ((q ^ (lane & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(h_cur[q].x), "=r"(h_cur[q].y), "=r"(h_cur[q].z), "=r"(h_cur[q].w)
                         : "r"(addr));
          }
          if (chunk + 1 < chunk_begin + kChunksPerWarp) {
            const int ncol0 = col0 + 32;
            const bool ok = row_ok && ncol0 + co_ck * 4 < N;
            const T* src = aux_in + (warp_row0 + co_row) * ld2 + 2 * ncol0 + co_ck * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              h_next[j] = ok ? __ldg(reinterpret_cast<const uint4*>(src + j * 4 * ld2)) : make_uint4(0, 0, 0, 0);
          }
        }
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the masked stores below
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
        if (EPI == EPI_DGLU) {
          // v = d(activated)[row, col0..col0+32); pre-activation (gate, up) pairs at columns 2*col
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // 8 pre-activation elements = 4 (gate, up) pairs per 16 bytes
            const uint32_t hw[4] = {h_cur[q].x, h_cur[q].y, h_cur[q].z, h_cur[q].w};
            float o[8];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const float2 gu = Elem<T>::unpack2(hw[p]);
              const float da = v[q * 4 + p];
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
            const uint32_t addr = dglu_stage + lane * 128 + ((q ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                         : "memory");
          }
          __syncwarp();
          const bool ok = row_ok && col0 + co_ck * 4 < N;
          T* dst = out + (warp_row0 + co_row) * ld2 + 2 * col0 + co_ck * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = j * 4 + co_row;
            uint4 u;
            const uint32_t addr = dglu_stage + r * 128 + ((co_ck ^ (r & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(addr));
            if (ok) *reinterpret_cast<uint4*>(dst + j * 4 * ld2) = u;
          }
          __syncwarp();
        }
      }
      }  // EPI != EPI_ACT
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
// host side
// ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// Tensor map over a row-major matrix (optionally batched): dims[0] is the contiguous one.
static int make_tmap(CUtensorMap* map, int dtype, const void* ptr, int rank, const uint64_t* dims,
                     const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return MOE_ERR_CUDA;
  }
  cuuint64_t gdim[3];
  cuuint64_t gstride[2];
  cuuint32_t bdim[3];
  cuuint32_t estr[3] = {1, 1, 1};
  uint64_t stride = 2;
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    stride *= dims[i];
    if (i < rank - 1) gstride[i] = stride;
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
  return MOE_OK;
}

// Process-wide cap on the CTAs of a grouped-GEMM launch (0 = none), see moe_set_gemm_grid_limit.
static std::atomic<int> g_grid_limit{0};

template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG, int CTAS>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<T, BN, A_K, B_K, EPI, KG, CTAS>;
  constexpr int smem = SmemPlan<BN, CTAS>::kTotal;
  static int grid_for_device[16] = {};  // 0 = not configured yet
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTAS > 1 ? 1 : 0;
  int grid = dev < 16 ? grid_for_device[dev] : 0;
  if (grid == 0) {
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
    if (const char* g = getenv("MOE_SM100_GRID")) {  // measurement aid: cap the number of resident workers
      const int want = atoi(g) / CTAS * CTAS;
      if (want > 0 && want < grid) grid = want;
    }
    if (dev < 16) grid_for_device[dev] = grid;
    if (getenv("MOE_SM100_DEBUG") != nullptr)
      fprintf(stderr, "[moe_sm100] grouped GEMM BN=%d CTAS=%d KG=%d: grid %d CTAs, %d bytes of shared memory\n", BN, CTAS,
              (int)KG, grid, smem);
  }
  {
    const int limit = g_grid_limit.load(std::memory_order_relaxed) / CTAS * CTAS;
    if (limit >= CTAS && limit < grid) grid = limit;
  }
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  MOE_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, args));
  return MOE_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Arrival counters of the wave barrier: a small ring in device memory; every launch that uses the barrier takes
// the next slot and zeroes it on its stream first.
constexpr int kWaveSlots = 256;
static __device__ uint32_t g_wave_counters[kWaveSlots];

static int next_wave_counter(cudaStream_t stream, uint32_t** out) {
  static uint32_t* base[16] = {};
  static unsigned next = 0;
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  uint32_t* b = dev < 16 ? base[dev] : nullptr;
  if (b == nullptr) {
    void* p = nullptr;
    MOE_CUDA(cudaGetSymbolAddress(&p, g_wave_counters));
    b = static_cast<uint32_t*>(p);
    if (dev < 16) base[dev] = b;
  }
  uint32_t* slot = b + (next++ % kWaveSlots);
  MOE_CUDA(cudaMemsetAsync(slot, 0, sizeof(uint32_t), stream));
  *out = slot;
  return MOE_OK;
}

// Row units per scheduling group; MOE_SM100_GROUP_M in the environment overrides it (measurement aid).
static int group_m_setting() {
  static int cached = 0;
  if (cached == 0) {
    const char* v = getenv("MOE_SM100_GROUP_M");
    const int n = v != nullptr ? atoi(v) : 0;
    cached = n > 0 ? n : kDefaultGroupM;
  }
  return cached;
}

// CTA pairs are the default; MOE_SM100_SINGLE_CTA=1 in the environment selects the one-CTA kernels
// (kept for comparison measurements).
static bool use_cta_pairs() {
  static int cached = -1;
  if (cached < 0) {
    const char* v = getenv("MOE_SM100_SINGLE_CTA");
    cached = (v != nullptr && v[0] == '1') ? 0 : 1;
  }
  return cached == 1;
}

template <typename T, int BN, int CTAS>
static int mgrouped_dispatch(const void* a, const void* w, int64_t padded_rows, int K, int N, int E, int w_transposed,
                             int epi, const GemmArgs& args, int dtype, cudaStream_t stream) {
  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)padded_rows};
    const uint32_t box[2] = {BK, BM};
    int rc = make_tmap(&ta, dtype, a, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  if (w_transposed) {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)E};
    const uint32_t box[3] = {BK, (uint32_t)(BN / CTAS), 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  } else {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)E};
    const uint32_t box[3] = {64, BK, 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  }
  if (epi == EPI_ACT) {
    return w_transposed ? launch<T, BN, true, true, EPI_ACT, false, CTAS>(ta, tb, args, stream)
                        : launch<T, BN, true, false, EPI_ACT, false, CTAS>(ta, tb, args, stream);
  } else if (epi == EPI_GLU) {
    return w_transposed ? launch<T, BN, true, true, EPI_GLU, false, CTAS>(ta, tb, args, stream)
                        : launch<T, BN, true, false, EPI_GLU, false, CTAS>(ta, tb, args, stream);
  } else if (epi == EPI_ACT_AUX) {
    return w_transposed ? launch<T, BN, true, true, EPI_ACT_AUX, false, CTAS>(ta, tb, args, stream)
                        : launch<T, BN, true, false, EPI_ACT_AUX, false, CTAS>(ta, tb, args, stream);
  }
  // EPI_DGLU is only used with the transposed weight (dAct = g @ W2^T).
  return launch<T, BN, true, true, EPI_DGLU, false, CTAS>(ta, tb, args, stream);
}

// 256-column tiles whenever there is more than one 128-column tile of work: with CTA pairs a 256 x 128 x 16 MMA
// takes ~144 cycles against ~158 for 256 x 256 x 16 (its operand reads from shared memory are the limit), so a
// half-empty last 256-column tile is far cheaper than narrow tiles throughout.
static int pick_bn(int N) { return N <= 128 ? 128 : 256; }

struct PushTarget {
  void* const* bases = nullptr;
  const int32_t* rank = nullptr;
  const int32_t* row = nullptr;
};

struct Chunk {
  int index = 0;
  int count = 1;
};

static int mgrouped_common(const void* a, const void* w, void* out, void* aux_out, const void* aux_in,
                           const PushTarget& push, const Chunk& chunk, const int32_t* mtile_expert,
                           const int32_t* tile_pairs, const int32_t* num_mtiles,
                           int64_t padded_rows, int K, int N, int E, int w_transposed, int epi, int act, int dtype,
                           int32_t* status, void* stream) {
  MOE_CHECK_ARG(a && w && (out || push.bases) && mtile_expert && num_mtiles, "grouped GEMM: null pointer argument");
  MOE_CHECK_ARG(aligned16(a) && aligned16(w) && aligned16(out) && aligned16(aux_out) && aligned16(aux_in),
                "grouped GEMM: pointers must be 16-byte aligned");
  MOE_CHECK_ARG(padded_rows > 0 && padded_rows % BM == 0, "grouped GEMM: padded_rows=%lld must be a positive multiple of %d",
                (long long)padded_rows, BM);
  MOE_CHECK_ARG(K > 0 && N > 0 && E > 0, "grouped GEMM: K=%d N=%d E=%d must be positive", K, N, E);
  if (K % 8 != 0 || N % 8 != 0 || (epi == EPI_GLU && N % 16 != 0)) {
    set_error("grouped GEMM: K=%d and N=%d must be multiples of 8 (16 for GLU outputs): rows must be 16-byte aligned", K, N);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(dtype == MOE_DTYPE_BF16 || dtype == MOE_DTYPE_F16, "grouped GEMM: unknown dtype %d", dtype);
  MOE_CHECK_ARG(chunk.count <= 1 || (tile_pairs != nullptr && chunk.index >= 0 && chunk.index < chunk.count),
                "grouped GEMM: chunk %d of %d needs tile_pairs and 0 <= index < count", chunk.index, chunk.count);
  GemmArgs args{};
  args.chunk_index = chunk.index;
  args.chunk_count = chunk.count;
  args.mtile_expert = mtile_expert;
  args.tile_pairs = tile_pairs;
  args.pair_prefix = tile_pairs != nullptr ? tile_pairs + padded_rows / BM : nullptr;
  {
    // Expert-aligned groups pay off when an expert has enough row-tile pairs to fill a group by itself
    // (measured: -36 % DRAM reads, +4 % speed at 8 pairs per expert; slower at ~4 pairs per expert, where
    // groups spanning several experts keep more CTA pairs on the same row tiles).
    const char* v = getenv("MOE_SM100_ALIGN_EXPERTS");
    const long long mean_rows = (padded_rows - static_cast<long long>(E) * (BM - 1)) / E;
    args.align_experts = tile_pairs == nullptr ? 0 : (v != nullptr ? atoi(v) : (mean_rows >= 6 * 2 * BM ? 1 : 0));
  }
  args.num_mtiles = num_mtiles;
  args.num_experts = E;
  args.n_dim = N;
  args.k_dim = K;
  args.out = out;
  args.aux_out = aux_out;
  args.aux_in = aux_in;
  args.push_bases = push.bases;
  args.push_rank = push.rank;
  args.push_row = push.row;
#ifdef MOE_GEMM_STATS
  {
    const char* sp = getenv("MOE_GEMM_STATS_PTR");
    args.stats = sp != nullptr ? reinterpret_cast<long long*>(strtoull(sp, nullptr, 0)) : nullptr;
  }
#endif
  args.act = act;
  args.group_m = group_m_setting();
  args.hint_weights_stream = getenv("MOE_SM100_L2_HINT") != nullptr ? 1 : 0;
  args.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    // The wave barrier cuts the DRAM reads of every M-grouped GEMM to about the algorithmic bytes (gate/up at
    // the Mixtral shape: 6.4 -> 2.1 GB), but only long contractions get faster (K = 14336: -1.2 %, K = 28672:
    // -2 %); at K = 4096 the synchronised bursts on shared tiles cost more than the re-reads (+6 %).  Hence
    // on for K >= 8192; MOE_SM100_WAVE_SYNC=0/1 overrides.
    const char* v = getenv("MOE_SM100_WAVE_SYNC");
    const bool on = v != nullptr ? atoi(v) != 0 : K >= 8192;
    const char* pv = getenv("MOE_SM100_WAVE_PERIOD");
    args.wave_period = pv != nullptr && atoi(pv) > 0 ? atoi(pv) : 1;
    args.wave_counter = nullptr;
    if (on) {
      const int rc = next_wave_counter(s, &args.wave_counter);
      if (rc != MOE_OK) return rc;
    }
  }
  const int bn = pick_bn(N);
  const bool pairs = tile_pairs != nullptr && use_cta_pairs();
#define MOE_MG(TYPE)                                                                                                  \
  (pairs ? (bn == 256 ? mgrouped_dispatch<TYPE, 256, 2>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s) \
                      : mgrouped_dispatch<TYPE, 128, 2>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s)) \
         : (bn == 256 ? mgrouped_dispatch<TYPE, 256, 1>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s) \
                      : mgrouped_dispatch<TYPE, 128, 1>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s)))
  if (dtype == MOE_DTYPE_BF16) return MOE_MG(__nv_bfloat16);
  return MOE_MG(__half);
#undef MOE_MG
}

template <typename T, int BN, int CTAS>
static int kgrouped_dispatch(const void* a, const void* b, int64_t padded_rows, int M, int N, const GemmArgs& args,
                             int dtype, cudaStream_t stream) {
  CUtensorMap ta, tb;
  const uint32_t box[2] = {64, BK};
  {
    const uint64_t dims[2] = {(uint64_t)M, (uint64_t)padded_rows};
    int rc = make_tmap(&ta, dtype, a, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)padded_rows};
    int rc = make_tmap(&tb, dtype, b, 2, dims, box);
    if (rc != MOE_OK) return rc;
  }
  return launch<T, BN, false, false, EPI_ACT, true, CTAS>(ta, tb, args, stream);
}

}  // namespace moe

using namespace moe;

extern "C" int moe_set_gemm_grid_limit(int max_ctas) {
  g_grid_limit.store(max_ctas > 0 ? max_ctas : 0, std::memory_order_relaxed);
  return MOE_OK;
}

extern "C" int moe_mgrouped_gemm(const void* a, const void* w, void* out, void* pre_act, const int32_t* mtile_expert,
                                 const int32_t* tile_pairs, const int32_t* num_mtiles, int64_t padded_rows, int K,
                                 int N, int num_experts, int w_transposed, int act, int dtype, int chunk_index,
                                 int chunk_count, int32_t* status, void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_NONE && act <= MOE_ACT_GEGLU, "moe_mgrouped_gemm: unknown activation %d", act);
  const bool glu = act == MOE_ACT_SWIGLU || act == MOE_ACT_GEGLU;
  if (!glu && (act == MOE_ACT_NONE || pre_act == nullptr)) pre_act = nullptr;  // nothing to save without an activation
  const int epi = glu ? EPI_GLU : (pre_act != nullptr ? EPI_ACT_AUX : EPI_ACT);
  return mgrouped_common(a, w, out, pre_act, nullptr, PushTarget{}, Chunk{chunk_index, chunk_count},
                         mtile_expert, tile_pairs, num_mtiles,
                         padded_rows, K, N, num_experts, w_transposed, epi, act, dtype, status, stream);
}

extern "C" int moe_mgrouped_gemm_dglu(const void* g, const void* w, const void* pre_act, void* d_pre,
                                      const int32_t* mtile_expert, const int32_t* tile_pairs,
                                      const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                      int act, int dtype, int chunk_index, int chunk_count, int32_t* status,
                                      void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_SILU && act <= MOE_ACT_GEGLU, "moe_mgrouped_gemm_dglu: activation %d has no derivative here", act);
  MOE_CHECK_ARG(pre_act != nullptr, "moe_mgrouped_gemm_dglu: pre_act is null");
  const bool glu = act == MOE_ACT_SWIGLU || act == MOE_ACT_GEGLU;
  return mgrouped_common(g, w, d_pre, nullptr, pre_act, PushTarget{}, Chunk{chunk_index, chunk_count}, mtile_expert,
                         tile_pairs, num_mtiles, padded_rows, K, N,
                         num_experts, 1, glu ? EPI_DGLU : EPI_ACT_AUX, act, dtype, status, stream);
}

extern "C" int moe_mgrouped_gemm_push(const void* a, const void* w, void* const* peer_bases, const int32_t* dest_rank,
                                      const int32_t* dest_row, const int32_t* mtile_expert, const int32_t* tile_pairs,
                                      const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                      int w_transposed, int dtype, int chunk_index, int chunk_count, int32_t* status,
                                      void* stream) {
  MOE_CHECK_ARG(peer_bases && dest_rank && dest_row, "moe_mgrouped_gemm_push: null pointer argument");
  PushTarget push;
  push.bases = peer_bases;
  push.rank = dest_rank;
  push.row = dest_row;
  return mgrouped_common(a, w, nullptr, nullptr, nullptr, push, Chunk{chunk_index, chunk_count}, mtile_expert, tile_pairs,
                         num_mtiles, padded_rows, K, N,
                         num_experts, w_transposed, EPI_ACT, MOE_ACT_NONE, dtype, status, stream);
}

extern "C" int moe_kgrouped_gemm(const void* a, const void* b, void* dw, const int32_t* pad_offsets,
                                 int64_t padded_rows, int M, int N, int num_experts, int dtype, int32_t* status,
                                 void* stream) {
  MOE_CHECK_ARG(a && b && dw && pad_offsets, "moe_kgrouped_gemm: null pointer argument");
  MOE_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(dw), "moe_kgrouped_gemm: pointers must be 16-byte aligned");
  MOE_CHECK_ARG(padded_rows > 0 && padded_rows % BM == 0, "moe_kgrouped_gemm: padded_rows=%lld must be a positive multiple of %d",
                (long long)padded_rows, BM);
  MOE_CHECK_ARG(M > 0 && N > 0 && num_experts > 0, "moe_kgrouped_gemm: M=%d N=%d E=%d must be positive", M, N, num_experts);
  if (M % 8 != 0 || N % 8 != 0) {
    set_error("moe_kgrouped_gemm: M=%d and N=%d must be multiples of 8", M, N);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(dtype == MOE_DTYPE_BF16 || dtype == MOE_DTYPE_F16, "moe_kgrouped_gemm: unknown dtype %d", dtype);
  GemmArgs args{};
  args.pad_offsets = pad_offsets;
  args.num_experts = num_experts;
  args.m_dim = M;
  args.n_dim = N;
  args.out = dw;
#ifdef MOE_GEMM_STATS
  {
    const char* sp = getenv("MOE_GEMM_STATS_PTR");
    args.stats = sp != nullptr ? reinterpret_cast<long long*>(strtoull(sp, nullptr, 0)) : nullptr;
  }
#endif
  args.act = MOE_ACT_NONE;
  args.group_m = group_m_setting();
  args.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bn = pick_bn(N);
  const bool pairs = use_cta_pairs();
#define MOE_KG(TYPE)                                                                              \
  (pairs ? (bn == 256 ? kgrouped_dispatch<TYPE, 256, 2>(a, b, padded_rows, M, N, args, dtype, s)  \
                      : kgrouped_dispatch<TYPE, 128, 2>(a, b, padded_rows, M, N, args, dtype, s)) \
         : (bn == 256 ? kgrouped_dispatch<TYPE, 256, 1>(a, b, padded_rows, M, N, args, dtype, s)  \
                      : kgrouped_dispatch<TYPE, 128, 1>(a, b, padded_rows, M, N, args, dtype, s)))
  if (dtype == MOE_DTYPE_BF16) return MOE_KG(__nv_bfloat16);
  return MOE_KG(__half);
#undef MOE_KG
}

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
// Roles inside a CTA (192 threads, one CTA per SM):
//   warp 0      : TMA producer  -- one lane issues cp.async.bulk.tensor tile loads into a
//                 ring of shared-memory stages (128-byte swizzle), signalled by mbarriers;
//   warp 1      : MMA issuer    -- one lane issues tcgen05.mma (128 x BN x 16, fp32
//                 accumulators in TMEM, two accumulator stages) and tcgen05.commit;
//   warps 2..5  : epilogue      -- tcgen05.ld the accumulator (each warp its 32-lane
//                 quadrant), apply the fused epilogue, store 16-byte vectors to global.
// The accumulator of tile i+1 is produced while tile i is being drained.
//
// Replaces the Triton kernels m_grouped_gemm_persistent_kernel / m_grouped_gemm_inner_kernel
// (reference: src/moe_explore/triton_kernels/m_grouped_gemm.py:33-267) and their epilogues
// (epilogue_split.py:4-44, triton_kernels/activation.py:5-36).
#include "common.cuh"

namespace moe {

constexpr int BM = 128;       // accumulator rows  (= TMEM lanes)
constexpr int BK = 64;        // K extent of one shared-memory stage: 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;    // K extent of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;
constexpr int kGroupM = 16;   // consecutive row tiles that share a sweep over column tiles (L2 reuse)
constexpr uint32_t kTmemCols = 512;

enum Epilogue : int { EPI_ACT = 0, EPI_GLU = 1, EPI_DGLU = 2 };

struct GemmArgs {
  // scheduling
  const int32_t* mtile_expert;  // M-grouped: expert of each 128-row tile
  const int32_t* num_mtiles;    // M-grouped: device scalar, tiles in use
  const int32_t* pad_offsets;   // K-grouped: padded row offsets [E+1]
  int32_t num_experts;
  int32_t m_dim;  // K-grouped: rows of each output matrix
  int32_t n_dim;  // accumulator columns (N of the contraction)
  int32_t k_dim;  // M-grouped: K of the contraction
  // epilogue
  void* out;           // EPI_ACT: [rows, N]; EPI_GLU: [rows, N/2]; EPI_DGLU: [rows, 2N]
  void* aux_out;       // EPI_GLU: un-activated product [rows, N] or null
  const void* aux_in;  // EPI_DGLU: saved un-activated product [rows, 2N]
  int32_t act;
  int32_t* status;
};

struct TileCoord {
  int m0;      // first accumulator row: padded row (M-grouped) or output-matrix row (K-grouped)
  int n0;      // first accumulator column
  int expert;
  int k_row0;  // K-grouped: first padded row of the contraction
  int kiters;  // number of BK-deep stages to contract
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
template <typename T, int BN, bool A_K, bool B_K>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  uint32_t d = 0;
  d |= 1u << 4;                       // D format: F32
  d |= Elem<T>::kUmmaFormat << 7;     // A format
  d |= Elem<T>::kUmmaFormat << 10;    // B format
  d |= (A_K ? 0u : 1u) << 15;         // A major: 0 = K, 1 = MN
  d |= (B_K ? 0u : 1u) << 16;         // B major
  d |= static_cast<uint32_t>(BN >> 3) << 17;
  d |= static_cast<uint32_t>(BM >> 4) << 24;
  return d;
}

template <int BN>
struct SmemPlan {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

template <bool KG>
__device__ __forceinline__ int total_tiles(const GemmArgs& args, int& mt, int& nt, int BN) {
  nt = (args.n_dim + BN - 1) / BN;
  if (KG) {
    mt = (args.m_dim + BM - 1) / BM;
    return args.num_experts * mt * nt;
  }
  mt = *args.num_mtiles;
  return mt * nt;
}

// Row tiles are walked in groups of kGroupM: inside a group every column tile is visited for
// all rows of the group before moving on, so concurrently running CTAs share operand tiles in L2.
template <bool KG>
__device__ __forceinline__ TileCoord decode_tile(int t, int mt, int nt, const GemmArgs& args, int BN) {
  TileCoord c;
  int expert = 0;
  if (KG) {
    expert = t / (mt * nt);
    t -= expert * (mt * nt);
  }
  const int per_group = kGroupM * nt;
  const int g = t / per_group;
  const int rem = t - g * per_group;
  const int m_first = g * kGroupM;
  const int gm = min(kGroupM, mt - m_first);
  const int n_idx = rem / gm;
  const int m_idx = m_first + (rem - n_idx * gm);
  c.m0 = m_idx * BM;
  c.n0 = n_idx * BN;
  if (KG) {
    c.expert = expert;
    c.k_row0 = args.pad_offsets[expert];
    c.kiters = (args.pad_offsets[expert + 1] - c.k_row0) / BK;  // padded ranges are multiples of 128
  } else {
    c.expert = args.mtile_expert[m_idx];
    c.k_row0 = 0;
    c.kiters = (args.k_dim + BK - 1) / BK;
  }
  return c;
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

template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs args) {
  using Plan = SmemPlan<BN>;
  constexpr int kStages = Plan::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;  // 128-byte swizzle atoms need 1024-byte alignment
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Plan::kStageBytes);
  const uint32_t full_bar = smem_u32(bars);                     // [kStages]
  const uint32_t empty_bar = smem_u32(bars + kStages);          // [kStages]
  const uint32_t tfull_bar = smem_u32(bars + 2 * kStages);      // [2]
  const uint32_t tempty_bar = smem_u32(bars + 2 * kStages + 2); // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int mt, nt;
  const int ntiles = total_tiles<KG>(args, mt, nt, BN);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        const TileCoord c = decode_tile<KG>(t, mt, nt, args, BN);
        for (int kb = 0; kb < c.kiters; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, args.status, DS_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t fb = full_bar + 8 * stage;
          const uint32_t sa = tiles_addr + stage * Plan::kStageBytes;
          const uint32_t sb = sa + Plan::kABytes;
          mbar_arrive_expect_tx(fb, Plan::kStageBytes);
          if (KG) {
            const int krow = c.k_row0 + kb * BK;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmap_a, c.m0 + 64 * j, krow, fb);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmap_b, c.n0 + 64 * j, krow, fb);
          } else {
            tma_load_2d(sa, &tmap_a, kb * BK, c.m0, fb);
            if (B_K) {
              tma_load_3d(sb, &tmap_b, kb * BK, c.n0, c.expert, fb);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * (BK * 128), &tmap_b, c.n0 + 64 * j, kb * BK, c.expert, fb);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Let copies that were already issued land before the CTA releases its shared memory.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<T, BN, A_K, B_K>();
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        const TileCoord c = decode_tile<KG>(t, mt, nt, args, BN);
        if (c.kiters == 0) continue;  // empty expert: the epilogue writes zeros on its own
        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, args.status, DS_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < c.kiters; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, args.status, DS_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = tiles_addr + stage * Plan::kStageBytes;
          const uint32_t sb = sa + Plan::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: step 16 elements (32 bytes) along the swizzled 128-byte row.
            // MN-major: step 16 k-rows of 128 bytes.
            const uint64_t da = A_K ? make_desc(sa + k * (UMMA_K * 2), 16, 1024)
                                    : make_desc(sa + k * (UMMA_K * 128), BK * 128, 1024);
            const uint64_t db = B_K ? make_desc(sb + k * (UMMA_K * 2), 16, 1024)
                                    : make_desc(sb + k * (UMMA_K * 128), BK * 128, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar + 8 * stage);  // frees the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull_bar + 8 * acc);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok || *abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    T* out = reinterpret_cast<T*>(args.out);
    T* aux_out = reinterpret_cast<T*>(args.aux_out);
    const T* aux_in = reinterpret_cast<const T*>(args.aux_in);
    const int N = args.n_dim;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const TileCoord c = decode_tile<KG>(t, mt, nt, args, BN);
      const bool have_acc = c.kiters != 0;
      if (have_acc) {
        if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, args.status, DS_TIMEOUT_EPILOGUE)) break;
        tc_fence_after();
      }
      const int row = c.m0 + row_in_tile;
      bool row_ok = true;
      long long out_row;  // row index into the output matrix
      if (KG) {
        row_ok = row < args.m_dim;
        out_row = static_cast<long long>(c.expert) * args.m_dim + row;
      } else {
        out_row = row;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        float v[32];
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
        const int col0 = c.n0 + chunk * 32;
        if (!row_ok || col0 >= N) {
          // nothing to store for this lane / column chunk
        } else if (EPI == EPI_ACT) {
          if (args.act == MOE_ACT_SILU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
          } else if (args.act == MOE_ACT_GELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_f(v[i]);
          }
          T* dst = out + out_row * N + col0;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (col0 + q * 8 < N) *reinterpret_cast<uint4*>(dst + q * 8) = pack8<T>(v + q * 8);
        } else if (EPI == EPI_GLU) {
          if (aux_out != nullptr) {
            T* dst = aux_out + out_row * N + col0;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (col0 + q * 8 < N) *reinterpret_cast<uint4*>(dst + q * 8) = pack8<T>(v + q * 8);
          }
          float g[16];
          if (args.act == MOE_ACT_GEGLU) {
#pragma unroll
            for (int i = 0; i < 16; ++i) g[i] = gelu_f(v[2 * i]) * v[2 * i + 1];
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) g[i] = silu_f(v[2 * i]) * v[2 * i + 1];
          }
          const int half_n = N >> 1;
          T* dst = out + out_row * half_n + (col0 >> 1);
#pragma unroll
          for (int q = 0; q < 2; ++q)
            if ((col0 >> 1) + q * 8 < half_n) *reinterpret_cast<uint4*>(dst + q * 8) = pack8<T>(g + q * 8);
        } else {  // EPI_DGLU: v = d(activated)[row, col0..col0+32); pre-activation pairs at columns 2*col
          const long long ld2 = 2ll * N;
          const T* src = aux_in + out_row * ld2 + 2 * col0;
          T* dst = out + out_row * ld2 + 2 * col0;
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // 8 pre-activation elements = 4 (gate, up) pairs per 16 bytes
            if (col0 + q * 4 >= N) continue;
            const uint4 h = *reinterpret_cast<const uint4*>(src + q * 8);
            const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
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
                const float s = sigmoidf_fast(gu.x);
                act_g = gu.x * s;
                dact_g = s * (1.0f + gu.x * (1.0f - s));
              }
              o[2 * p] = da * gu.y * dact_g;
              o[2 * p + 1] = da * act_g;
            }
            *reinterpret_cast<uint4*>(dst + q * 8) = pack8<T>(o);
          }
        }
      }
      if (have_acc) {
        tc_fence_before();
        mbar_arrive(tempty_bar + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
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

template <typename T, int BN, bool A_K, bool B_K, int EPI, bool KG>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args, int grid, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<T, BN, A_K, B_K, EPI, KG>;
  constexpr int smem = SmemPlan<BN>::kTotal;
  static bool configured[16] = {};
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    MOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  } else if (dev >= 16) {
    MOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  }
  kernel<<<grid, kThreads, smem, stream>>>(ta, tb, args);
  MOE_CUDA(cudaGetLastError());
  return MOE_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int BN>
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
    const uint32_t box[3] = {BK, (uint32_t)BN, 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  } else {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)E};
    const uint32_t box[3] = {64, BK, 1};
    int rc = make_tmap(&tb, dtype, w, 3, dims, box);
    if (rc != MOE_OK) return rc;
  }
  const int grid = sm_count();
  if (epi == EPI_ACT) {
    return w_transposed ? launch<T, BN, true, true, EPI_ACT, false>(ta, tb, args, grid, stream)
                        : launch<T, BN, true, false, EPI_ACT, false>(ta, tb, args, grid, stream);
  } else if (epi == EPI_GLU) {
    return w_transposed ? launch<T, BN, true, true, EPI_GLU, false>(ta, tb, args, grid, stream)
                        : launch<T, BN, true, false, EPI_GLU, false>(ta, tb, args, grid, stream);
  }
  // EPI_DGLU is only used with the transposed weight (dAct = g @ W2^T).
  return launch<T, BN, true, true, EPI_DGLU, false>(ta, tb, args, grid, stream);
}

static int pick_bn(int N) { return (N % 256 == 0 || N % 128 != 0) ? 256 : 128; }

static int mgrouped_common(const void* a, const void* w, void* out, void* aux_out, const void* aux_in,
                           const int32_t* mtile_expert, const int32_t* num_mtiles, int64_t padded_rows, int K, int N,
                           int E, int w_transposed, int epi, int act, int dtype, int32_t* status, void* stream) {
  MOE_CHECK_ARG(a && w && out && mtile_expert && num_mtiles, "grouped GEMM: null pointer argument");
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
  GemmArgs args{};
  args.mtile_expert = mtile_expert;
  args.num_mtiles = num_mtiles;
  args.num_experts = E;
  args.n_dim = N;
  args.k_dim = K;
  args.out = out;
  args.aux_out = aux_out;
  args.aux_in = aux_in;
  args.act = act;
  args.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bn = pick_bn(N);
  if (dtype == MOE_DTYPE_BF16) {
    return bn == 256 ? mgrouped_dispatch<__nv_bfloat16, 256>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s)
                     : mgrouped_dispatch<__nv_bfloat16, 128>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s);
  }
  return bn == 256 ? mgrouped_dispatch<__half, 256>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s)
                   : mgrouped_dispatch<__half, 128>(a, w, padded_rows, K, N, E, w_transposed, epi, args, dtype, s);
}

template <typename T, int BN>
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
  return launch<T, BN, false, false, EPI_ACT, true>(ta, tb, args, sm_count(), stream);
}

}  // namespace moe

using namespace moe;

extern "C" int moe_mgrouped_gemm(const void* a, const void* w, void* out, void* pre_act, const int32_t* mtile_expert,
                                 const int32_t* num_mtiles, int64_t padded_rows, int K, int N, int num_experts,
                                 int w_transposed, int act, int dtype, int32_t* status, void* stream) {
  MOE_CHECK_ARG(act >= MOE_ACT_NONE && act <= MOE_ACT_GEGLU, "moe_mgrouped_gemm: unknown activation %d", act);
  const bool glu = act == MOE_ACT_SWIGLU || act == MOE_ACT_GEGLU;
  return mgrouped_common(a, w, out, glu ? pre_act : nullptr, nullptr, mtile_expert, num_mtiles, padded_rows, K, N,
                         num_experts, w_transposed, glu ? EPI_GLU : EPI_ACT, act, dtype, status, stream);
}

extern "C" int moe_mgrouped_gemm_dglu(const void* g, const void* w, const void* pre_act, void* d_pre,
                                      const int32_t* mtile_expert, const int32_t* num_mtiles, int64_t padded_rows,
                                      int K, int N, int num_experts, int act, int dtype, int32_t* status,
                                      void* stream) {
  MOE_CHECK_ARG(act == MOE_ACT_SWIGLU || act == MOE_ACT_GEGLU, "moe_mgrouped_gemm_dglu: activation %d is not a GLU", act);
  MOE_CHECK_ARG(pre_act != nullptr, "moe_mgrouped_gemm_dglu: pre_act is null");
  return mgrouped_common(g, w, d_pre, nullptr, pre_act, mtile_expert, num_mtiles, padded_rows, K, N, num_experts, 1,
                         EPI_DGLU, act, dtype, status, stream);
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
  args.act = MOE_ACT_NONE;
  args.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bn = pick_bn(N);
  if (dtype == MOE_DTYPE_BF16) {
    return bn == 256 ? kgrouped_dispatch<__nv_bfloat16, 256>(a, b, padded_rows, M, N, args, dtype, s)
                     : kgrouped_dispatch<__nv_bfloat16, 128>(a, b, padded_rows, M, N, args, dtype, s);
  }
  return bn == 256 ? kgrouped_dispatch<__half, 256>(a, b, padded_rows, M, N, args, dtype, s)
                   : kgrouped_dispatch<__half, 128>(a, b, padded_rows, M, N, args, dtype, s);
}

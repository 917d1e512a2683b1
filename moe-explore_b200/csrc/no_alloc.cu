// moe_routing_metadata_static: the routing-metadata entry point for callers that cannot
// allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- inside a region whose memory
// is owned by a fixed-size arena handed over at start-up (inference servers that pre-size every
// buffer), plugin hosts that give an operator its inputs and outputs and nothing else, or a
// latency-critical loop that must not take the allocator's locks.  Such callers still own the
// inputs and outputs; the only thing they cannot provide is the counting sort's scratch
// (per-chunk histograms and offsets).  Here that scratch lives in a file-scope __device__ array
// that every GPU loading this library carries until the process exits.
//
// Limits and rules
//   * the array holds kStaticScratchBytes (1 MiB); a problem whose scratch requirement
//     (moe_routing_workspace_bytes) is larger is rejected with MOE_ERR_UNSUPPORTED;
//   * every call on a device shares the one array: two calls that overlap on the GPU (different
//     streams, or different host threads) race on it -- serialise them;
//   * the array keeps whatever the previous call left in it; nothing in it has to start at zero,
//     because the histogram kernel overwrites every word the later kernels read;
//   * the first call on each device looks up the array's device address (one
//     cudaGetSymbolAddress, no allocation); make that first call outside any stream capture.
#include "common.cuh"

#include <atomic>

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_routing_scratch[kStaticScratchBytes];

// Device address of g_routing_scratch on each device.  In host code the symbol's name is only a
// handle: the address a kernel can use has to be asked for, per device, with that device current.
// Atomic slots: two host threads making a device's first call together both look the address up
// and store the same value.
std::atomic<void*> g_scratch_ptr[kMaxDevices];

int scratch_for_current_device(void** out) {
  int dev = -1;
  MOE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    moe::set_error("moe_routing_metadata_static: device ordinal %d is outside the supported range [0, %d)", dev,
                   kMaxDevices);
    return MOE_ERR_UNSUPPORTED;
  }
  void* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    MOE_CUDA(cudaGetSymbolAddress(&p, g_routing_scratch));
    g_scratch_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return MOE_OK;
}

}  // namespace

extern "C" size_t moe_routing_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int moe_routing_metadata_static(const int64_t* expert_idx, int64_t num_rows, int num_experts,
                                           int32_t* group_indices, int64_t* perm, int32_t* pad_offsets,
                                           int32_t* row_src, int32_t* dst_row, int32_t* mtile_expert,
                                           int32_t* tile_pairs, int32_t* num_mtiles, int32_t* status,
                                           void* stream) {
  if (num_rows < 0 || num_experts <= 0) {
    moe::set_error("moe_routing_metadata_static: bad sizes num_rows=%lld num_experts=%d", (long long)num_rows,
                   num_experts);
    return MOE_ERR_INVALID;
  }
  const size_t need = moe_routing_workspace_bytes(num_rows, num_experts);
  if (need > kStaticScratchBytes) {
    moe::set_error(
        "moe_routing_metadata_static: num_rows=%lld with num_experts=%d needs %zu bytes of scratch; the built-in "
        "scratch holds %zu (use moe_routing_metadata with a caller-owned workspace)",
        (long long)num_rows, num_experts, need, kStaticScratchBytes);
    return MOE_ERR_UNSUPPORTED;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != MOE_OK) return rc;
  return moe_routing_metadata(expert_idx, num_rows, num_experts, group_indices, perm, pad_offsets, row_src, dst_row,
                              mtile_expert, tile_pairs, num_mtiles, status, scratch, kStaticScratchBytes, stream);
}

// Library-wide host helpers behind the C ABI: thread-local error text, device queries and
// the device status word check.
#include "common.cuh"

#include <string.h>

#include <atomic>

namespace moe {

static std::atomic<long long> g_wait_limit{kDefaultWaitLimitCycles};
long long wait_limit_cycles() { return g_wait_limit.load(std::memory_order_relaxed); }

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return MOE_ERR_CUDA;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 64) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace moe

using namespace moe;

extern "C" const char* moe_last_error(void) { return g_error; }

extern "C" int moe_query_device(int device, int* sm_count_out, int* cc_major, int* cc_minor) {
  int n = 0, major = 0, minor = 0;
  MOE_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  MOE_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  MOE_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (sm_count_out) *sm_count_out = n;
  if (cc_major) *cc_major = major;
  if (cc_minor) *cc_minor = minor;
  if (major != 10) {
    set_error("device %d has compute capability %d.%d; this library contains sm_100a code only", device, major, minor);
    return MOE_ERR_UNSUPPORTED;
  }
  return MOE_OK;
}

extern "C" int moe_check_status(const int32_t* status, void* stream) {
  MOE_CHECK_ARG(status != nullptr, "moe_check_status: status is null");
  int32_t host = 0;
  MOE_CUDA(cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  MOE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (host == 0) return MOE_OK;
  if (host == DS_BAD_EXPERT_ID) {
    set_error("routing metadata saw an expert id outside [0, num_experts); such rows were dropped");
    return MOE_ERR_INVALID;
  }
  if (host == DS_BAD_LAYOUT) {
    set_error("routing metadata does not describe the rows it was used with (a group prefix that is not a prefix of "
              "num_rows, or padded_rows differing from the bound the metadata was built with)");
    return MOE_ERR_INVALID;
  }
  if (host == DS_WAVE_FALLBACK) {
    set_error("the wave barrier of a grouped GEMM ran out (its workers were not all resident); that launch finished "
              "with unsynchronised scheduling and its results are valid");
    return MOE_ERR_TIMEOUT;
  }
  set_error("a device-side bounded wait ran out (code %d: 1 = TMA producer, 2 = MMA issuer, 3 = epilogue); the outputs "
            "of that launch are incomplete", host);
  return MOE_ERR_TIMEOUT;
}

extern "C" int moe_read_status(const int32_t* status, int32_t* code, int reset, void* stream) {
  MOE_CHECK_ARG(status != nullptr && code != nullptr, "moe_read_status: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MOE_CUDA(cudaMemcpyAsync(code, status, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  if (reset) MOE_CUDA(cudaMemsetAsync(const_cast<int32_t*>(status), 0, sizeof(int32_t), s));
  MOE_CUDA(cudaStreamSynchronize(s));
  return MOE_OK;
}

extern "C" size_t moe_gemm_options_size(void) { return sizeof(moe_gemm_options); }

extern "C" int moe_set_wait_limit_cycles(int64_t cycles) {
  g_wait_limit.store(cycles > 0 ? cycles : kDefaultWaitLimitCycles, std::memory_order_relaxed);
  return MOE_OK;
}

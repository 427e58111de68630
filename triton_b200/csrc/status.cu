// Status word, TMA descriptor encoder and device-property cache (host side).
#include <stdio.h>
#include <mutex>

#include "common.cuh"
#include "host_common.h"

namespace tb200 {

// One word per device that loads this library. Kernels write a non-zero code here when a
// bounded wait gives up; tb200_check() reads and clears it.
__device__ int g_status_word = 0;

static constexpr int kMaxDevices = 64;
static int* g_status_ptrs[kMaxDevices] = {};
static int g_sm_counts[kMaxDevices] = {};
static std::mutex g_mu;

int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status_ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_ptrs[dev] = static_cast<int*>(p);
  }
  return g_status_ptrs[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_sm_counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sm_counts[dev] = n;
  }
  return g_sm_counts[dev];
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = []() -> EncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                CUtensorMapL2promotion promo) {
  EncodeFn fn = get_encode_fn();
  if (!fn || rank < 1 || rank > 5) return TB200_ERR_TMAP;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a host thread that has made no runtime call yet (e.g. an autograd worker) has no current
    // context: bind the device's primary context and encode again
    cudaFree(nullptr);
    r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_TMAP;
}

// One thread waits, through the same bounded wait every kernel of the library uses, on an mbarrier
// that nobody arrives on. No copy and no MMA is in flight, so when the limit runs out the thread
// records WAIT_SELFTEST in the status word and the block simply returns.
__global__ void selftest_wait_kernel(int* status, unsigned long long limit_ns, int* waited_out) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    const bool done = mbar_wait_limit(&bar, 0, status, WAIT_SELFTEST, limit_ns);
    if (waited_out) *waited_out = done ? 1 : 0;
  }
}

}  // namespace tb200

extern "C" int tb200_selftest_wait(uint64_t limit_ns, int* completed, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return TB200_ERR_BAD_ARG;  // at most one second
  int* p = tb200::status_ptr();
  if (!p) return TB200_ERR_CUDA;
  tb200::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, limit_ns, completed);
  return tb200::cuda_err(cudaGetLastError());
}

extern "C" int tb200_check(void* stream) {
  int* p = tb200::status_ptr();
  if (!p) return TB200_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  if (cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return TB200_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return TB200_ERR_CUDA;
  if (v == 0) return TB200_OK;
  cudaMemsetAsync(p, 0, sizeof(int), s);
  cudaStreamSynchronize(s);
  return TB200_ERR_TIMEOUT;
}

extern "C" int tb200_last_status_code(void) {
  int* p = tb200::status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

extern "C" const char* tb200_error_string(int code) {
  switch (code) {
    case TB200_OK: return "ok";
    case TB200_ERR_BAD_ARG: return "bad argument (null pointer, negative size, misaligned base or stride)";
    case TB200_ERR_UNSUPPORTED: return "unsupported shape, dtype or layout for this kernel";
    case TB200_ERR_CUDA: return "CUDA runtime call failed";
    case TB200_ERR_TIMEOUT: return "a device-side wait timed out; results of the last launches are invalid";
    case TB200_ERR_TMAP: return "TMA descriptor encoding failed";
    case TB200_ERR_TOO_LARGE: return "size exceeds the fixed capacity of this entry point";
    default: return "unknown error";
  }
}

extern "C" int tb200_version(void) { return 1; }

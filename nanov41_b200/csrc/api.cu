// Library identification and the device status word reader of the C ABI.
#include <cuda_runtime.h>

#include "../../include/nanov41_b200.h"

#include <atomic>

#include "util.cuh"

namespace nv41 {
static std::atomic<int> g_gemm_cta_limit{0};
int gemm_cta_limit() { return g_gemm_cta_limit.load(std::memory_order_relaxed); }
}  // namespace nv41

extern "C" int nv41_abi_version(void) { return 101; }

extern "C" int nv41_set_gemm_cta_limit(int max_ctas) {
  if (max_ctas < 0) return NV41_ERR_INVALID;
  nv41::g_gemm_cta_limit.store(max_ctas, std::memory_order_relaxed);
  return NV41_OK;
}

extern "C" int nv41_status_read(const unsigned* status, unsigned* raw_host, void* stream) {
  if (!status) return NV41_ERR_INVALID;
  unsigned v = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&v, status, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return NV41_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return NV41_ERR_CUDA;
  if (raw_host) *raw_host = v;
  return v == 0u ? NV41_OK : NV41_ERR_TIMEOUT;
}

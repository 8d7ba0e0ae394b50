// Host-side helpers shared by the translation units of the C-ABI library.
#pragma once
#include <cuda_runtime.h>

#include "../../include/nanov41_b200.h"

namespace nv41 {

// Status of the launch that was just enqueued (never synchronises).
inline int launch_status() {
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? NV41_OK : NV41_ERR_CUDA;
}

// Upper bound on the CTAs of the persistent grouped GEMMs (0 = one per SM); see
// nv41_set_gemm_cta_limit.
int gemm_cta_limit();

// Grid of a persistent GEMM on a device with `sms` SMs.
inline int persistent_grid(int sms) {
  const int lim = gemm_cta_limit();
  return (lim > 0 && lim < sms) ? lim : sms;
}

}  // namespace nv41

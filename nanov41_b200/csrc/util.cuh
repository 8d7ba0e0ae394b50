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

}  // namespace nv41

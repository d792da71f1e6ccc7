// SPDX-License-Identifier: MIT
//
// Kernel launch helper with programmatic dependent launch: a kernel launched
// through launch_k may begin (block scheduling, barrier/TMEM set-up, weight
// prefetch) while its predecessor in the stream is still draining.  Every
// such kernel executes pdl_wait() before it touches memory that an earlier
// kernel writes or reads, which orders it after the predecessor's completion.
// BL_PDL=0 turns the attribute off (plain stream order).
#pragma once

#include <cuda_runtime.h>
#include <stdlib.h>

namespace bl {

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("BL_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace bl

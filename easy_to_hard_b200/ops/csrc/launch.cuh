// Kernel launch helper with optional programmatic dependent launch (PDL).
//
// With PDL on, a kernel may start (set up barriers, tensor memory, descriptors) while its
// predecessor in the stream is still draining; it must execute griddepcontrol.wait before it
// touches any global memory. Every kernel launched through this helper does so first thing
// (pdl_wait_prior in ptx.cuh), which is a no-op when the launch carries no PDL attribute. The
// switch is process-wide (e2h_set_pdl) and is what the decode engine turns on while it records
// its CUDA graph, where ~230 short kernels run back to back.
#pragma once
#include <cuda_runtime.h>
#include <string.h>

namespace e2h {

inline int g_pdl = 0;

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (g_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace e2h

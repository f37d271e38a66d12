// Host-side launch helper: one place that sets the launch attributes used by every kernel
// of the library (programmatic dependent launch, cooperative launch for emulation).
#pragma once
#include <cuda_runtime.h>

namespace mcb {

// pdl != 0       : the kernel may start while its predecessor in the stream drains; the
//                  kernel itself calls griddepcontrol.wait before touching memory.
// cooperative    : all blocks must be co-resident (blocks of different emulated ranks wait
//                  on one another inside one launch).
template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         int pdl, bool cooperative, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (pdl) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cooperative) {
    attrs[n].id = cudaLaunchAttributeCooperative;
    attrs[n].val.cooperative = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace mcb

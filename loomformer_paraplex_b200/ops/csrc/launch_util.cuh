// Programmatic dependent launch for chains of short kernels.
//
// A kernel launched through launch_pdl may become resident while the previous kernel of its stream is still running
// (once every block of that kernel has executed pdl_trigger or exited).  Whatever it does before pdl_wait must not
// touch memory that an earlier kernel of the stream writes (weights, constants and its own shared memory are fine);
// pdl_wait returns when the previous kernel has completed and its writes are visible.  Every kernel launched this way
// executes pdl_wait on all paths, so "this kernel has completed" keeps implying "everything before it has completed".
// Kernels launched the ordinary way may still call pdl_trigger: it only lets a dependent start its prologue early.
// LOOM_PDL=0 turns the launch attribute off (the device-side calls are then no-ops).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace loom {

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("LOOM_PDL"); v = (e != nullptr && e[0] == '0') ? 0 : 1; }
  return v != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t shm, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = shm; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace loom

// Host-side helpers shared by the C-ABI entry points: error text, argument checks, per-device properties and the
// device status word that kernels set when a bounded wait runs out.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

namespace st {
int fail(const char* fmt, ...);                 // stores the message for st_last_error(), returns 1
int cuda_fail(cudaError_t e, const char* what); // 0 when e == cudaSuccess
int sm_count();                                 // SMs of the current device (cached)
int* status_ptr();                              // device address of the current device's status word array
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool pdl_enabled();                             // STATETREE_PDL=0 turns programmatic dependent launch off

// Launches `kernel` so that it may start under the tail of its predecessor in the stream (programmatic dependent
// launch): the set-up and scheduling of a short kernel then overlap the previous kernel instead of following it.
// Every kernel launched this way executes griddepcontrol.wait before it touches anything a predecessor wrote.
template <typename... Params, typename... Args>
inline int launch(const char* who, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cuda_fail(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...), who);
}
}  // namespace st

#define ST_REQUIRE(cond, ...) do { if (!(cond)) return st::fail(__VA_ARGS__); } while (0)
#define ST_LAUNCH_CHECK(what) do { if (int e_ = st::cuda_fail(cudaGetLastError(), what)) return e_; } while (0)

// Host-side helpers shared by the C-ABI entry points: error text, argument checks, per-device properties and the
// device status word that kernels set when a bounded wait runs out.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace st {
int fail(const char* fmt, ...);                 // stores the message for st_last_error(), returns 1
int cuda_fail(cudaError_t e, const char* what); // 0 when e == cudaSuccess
int sm_count();                                 // SMs of the current device (cached)
int* status_ptr();                              // device address of the current device's status word array
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace st

#define ST_REQUIRE(cond, ...) do { if (!(cond)) return st::fail(__VA_ARGS__); } while (0)
#define ST_LAUNCH_CHECK(what) do { if (int e_ = st::cuda_fail(cudaGetLastError(), what)) return e_; } while (0)

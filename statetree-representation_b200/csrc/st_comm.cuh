// Layout of a rank's communication buffer (plain device memory, exported to the peers of the node as a CUDA IPC
// handle) and the system-scope loads / stores the kernels use on it.  Shared by st_comm.cu (all-reduce kernels) and
// st_gemv.cu (the row-parallel GEMV that sums its output over the ranks itself).
//
//     flags  uint32 [MAX_RANKS][MAX_CTAS]   all-reduce: flags[p][c] = last epoch in which rank p's CTA c delivered here
//     epoch  uint32 [MAX_CTAS]              all-reduce: calls made so far, per CTA slot
//     gemv   uint32 [2]                     fused GEMV: calls made so far; CTAs of the current call that have finished
//     data   2 x MAX_RANKS x MAX_BYTES      all-reduce: the partial sums of every rank, double-buffered by epoch parity
//     recv   2 x MAX_RANKS x RECV_VALUES    fused GEMV: fp32 tile sums of every rank, one word per output value,
//                                           double-buffered by call parity; a word holds all ones until its value lands
#pragma once
#include <stdint.h>

namespace st {
constexpr int MAX_RANKS = 8;
constexpr int MAX_CTAS = 64;
constexpr long long SLOT_BYTES = 16 << 10;                            // all-reduce: per CTA and call
constexpr long long MAX_BYTES = MAX_CTAS * SLOT_BYTES;                // all-reduce: per call (1 MiB)
constexpr long long RECV_VALUES = 128 << 10;                          // fused GEMV: padded output values per call
constexpr size_t OFF_EPOCH = (size_t)MAX_RANKS * MAX_CTAS * 4;
constexpr size_t OFF_GEMV = OFF_EPOCH + MAX_CTAS * 4;                 // 2304
constexpr size_t OFF_DATA = OFF_GEMV + 256;                           // 2560: 256-byte aligned
constexpr size_t OFF_RECV = OFF_DATA + 2 * (size_t)MAX_RANKS * (size_t)MAX_BYTES;
constexpr size_t RECV_BYTES = 2 * (size_t)MAX_RANKS * (size_t)RECV_VALUES * 4;
constexpr size_t COMM_BYTES = OFF_RECV + RECV_BYTES;
constexpr uint32_t RECV_EMPTY = 0xFFFFFFFFu;                          // a NaN pattern no fp32 addition produces

struct Peers {
  uint8_t* buf[MAX_RANKS];                                            // buf[rank] is the local buffer
};

long long comm_wait_ns();                                             // the wall-time bound of cross-GPU waits

#ifdef __CUDACC__
__device__ __forceinline__ long long now_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {   // never served from a stale local cache line
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// fused GEMV: where rank `src` delivers value `idx` of a call with parity `half`, inside the buffer `buf`
__device__ __forceinline__ uint32_t* recv_word(uint8_t* buf, int half, int src, long long idx) {
  return reinterpret_cast<uint32_t*>(buf + OFF_RECV) + ((size_t)half * MAX_RANKS + src) * (size_t)RECV_VALUES + idx;
}
#endif
}  // namespace st

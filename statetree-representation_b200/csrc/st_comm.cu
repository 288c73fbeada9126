// Tensor-parallel exchange over NVLink peer memory: a one-shot all-reduce of the small BF16 partial outputs of the
// row-parallel linears (o and down projections: batch x hidden values per call), optionally fused with the residual
// add and RMSNorm that consume it in a decode step.
//
// Every rank owns one communication buffer (layout in st_comm.cuh): per (source rank, CTA slot) a flag word and a data
// region, double-buffered by the parity of that slot's epoch (all ranks make the same calls).
// One call, CTA c of rank r: PUSH slice c of the local partials into region (r, c) of every rank's buffer (remote
// stores; the own copy is a local store), system-scope fence, store the epoch into flags[r][c] of every peer; wait until
// flags[p][c] of the own buffer reach the epoch for every p (local loads; bounded); add the world copies of slice c in
// rank order from the OWN buffer (local loads, fp32) and write the BF16 result.  The data crosses NVLink once, as
// stores, and nobody waits on a remote load.  The double buffer makes a second barrier unnecessary: a rank overwrites
// region (r, c) of a peer two calls later, after a wait that the peer satisfies only at the start of its next call,
// when it has finished reading the earlier one.
// The wait is bounded by wall time (st_comm_set_timeout_ms, 20 s unless set); when it runs out the kernel records
// ERR_WAIT_PEER in the device status word and leaves its output unwritten: the step's result is then invalid and the
// host must check st_device_status() before it trusts it.  The reference has no communication code (vLLM adds NCCL
// collectives around it).
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/statetree_b200.h"
#include "st_comm.cuh"
#include "st_common.cuh"
#include "st_host.h"

namespace {
using namespace st;

long long g_wait_ns = 20000000000ll;                                  // st_comm_set_timeout_ms

__device__ __forceinline__ uint8_t* slot_data(uint8_t* buf, int half, int src_rank, int cta) {
  return buf + OFF_DATA + ((size_t)half * MAX_RANKS + src_rank) * MAX_BYTES + (size_t)cta * SLOT_BYTES;
}

// Delivers the len bytes at src (16-byte units, len <= SLOT_BYTES) as slot `cta` of this call to every rank and returns
// once every rank's slot `cta` has arrived here.  Called by all threads of the CTA; returns the data half to read from
// (in the own buffer), or -1 after a timeout.
__device__ int publish_and_wait(const Peers& P, int rank, int world, const uint8_t* src, size_t len, int cta, int* status,
                                long long wait_ns) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  uint8_t* mine = P.buf[rank];
  if (threadIdx.x == 0) {
    uint32_t* ep = reinterpret_cast<uint32_t*>(mine + OFF_EPOCH) + cta;
    s_epoch = *ep + 1u;
    *ep = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int half = (int)(epoch & 1u);
  for (size_t i = (size_t)threadIdx.x * 16; i < len; i += (size_t)blockDim.x * 16) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i);
    for (int p = 0; p < world; ++p) *reinterpret_cast<uint4*>(slot_data(P.buf[p], half, rank, cta) + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const int p = threadIdx.x;
    st_release_sys(reinterpret_cast<uint32_t*>(P.buf[p]) + rank * MAX_CTAS + cta, epoch);      // "rank's slot is there"
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine) + p * MAX_CTAS + cta;
    const long long t0 = now_ns();
    // epochs only grow; the signed difference also survives the 32-bit wrap
    while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
      if (now_ns() - t0 > wait_ns) {
        atomicExch(status, ERR_WAIT_PEER);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok ? half : -1;
}

// out = sum over ranks of the BF16 vectors `in` (n elements, a multiple of 8); grid <= MAX_CTAS
__global__ void __launch_bounds__(256) allreduce_kernel(const Peers P, int rank, int world, const uint16_t* in,
                                                        uint16_t* out, long long n, int* status, long long wait_ns) {
  pdl_wait();
  pdl_launch_dependents();
  const long long vecs = n / 8, per = (vecs + gridDim.x - 1) / gridDim.x;
  const long long v0 = (long long)blockIdx.x * per, v1 = min(vecs, v0 + per);
  const size_t off = (size_t)v0 * 16, len = v1 > v0 ? (size_t)(v1 - v0) * 16 : 0;
  const int h = publish_and_wait(P, rank, world, reinterpret_cast<const uint8_t*>(in) + off, len, blockIdx.x, status, wait_ns);
  uint8_t* mine = P.buf[rank];
  if (h < 0) return;
  for (size_t i = (size_t)threadIdx.x * 16; i < len; i += (size_t)blockDim.x * 16) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < world; ++p) {
      const uint4 v = ld_peer16(slot_data(mine, h, p, blockIdx.x) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(out) + off + i) = o;
  }
}

__device__ __forceinline__ float block_sum(float v, float* part) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += part[i];
  return tot;
}

// One CTA per row: delta_sum = sum over ranks of `delta` rows (rank order, fp32, rounded to BF16 as the separate
// all-reduce would); x += delta_sum (BF16 residual stream); out = RMSNorm(x) * w.  cols <= 8192, a multiple of 8.
__global__ void __launch_bounds__(512) allreduce_add_rmsnorm_kernel(const Peers P, int rank, int world, uint16_t* x,
                                                                    const uint16_t* delta, const uint16_t* w,
                                                                    uint16_t* out, int cols, float eps, int* status,
                                                                    long long wait_ns) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float part[16];
  const size_t rowb = (size_t)blockIdx.x * cols * 2;
  const int h = publish_and_wait(P, rank, world, reinterpret_cast<const uint8_t*>(delta) + rowb, (size_t)cols * 2,
                                 blockIdx.x, status, wait_ns);
  if (h < 0) return;
  uint8_t* mine = P.buf[rank];
  float f[2][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int c = (threadIdx.x + k * 512) * 8;
    if (c < cols) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int p = 0; p < world; ++p) {
        const uint4 v = ld_peer16(slot_data(mine, h, p, blockIdx.x) + (size_t)c * 2);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += __uint_as_float(u[q] << 16);
          acc[2 * q + 1] += __uint_as_float(u[q] & 0xFFFF0000u);
        }
      }
      const uint4 xv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(x) + rowb + (size_t)c * 2);
      const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
      uint32_t so[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t d = pack_bf16(acc[2 * q], acc[2 * q + 1]);      // the all-reduced delta is a BF16 tensor
        const uint32_t s = pack_bf16(__uint_as_float(xs[q] << 16) + __uint_as_float(d << 16),
                                     __uint_as_float(xs[q] & 0xFFFF0000u) + __uint_as_float(d & 0xFFFF0000u));
        so[q] = s;
        f[k][2 * q] = __uint_as_float(s << 16);
        f[k][2 * q + 1] = __uint_as_float(s & 0xFFFF0000u);
        ss += f[k][2 * q] * f[k][2 * q] + f[k][2 * q + 1] * f[k][2 * q + 1];
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(x) + rowb + (size_t)c * 2) = make_uint4(so[0], so[1], so[2], so[3]);
    }
  }
  const float r = rsqrtf(block_sum(ss, part) / (float)cols + eps);
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int c = (threadIdx.x + k * 512) * 8;
    if (c < cols) {
      const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
      const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t nrm = pack_bf16(f[k][2 * q] * r, f[k][2 * q + 1] * r);        // normalised value rounded, then scaled
        o[q] = pack_bf16(__uint_as_float(nrm << 16) * __uint_as_float(ws[q] << 16),
                         __uint_as_float(nrm & 0xFFFF0000u) * __uint_as_float(ws[q] & 0xFFFF0000u));
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(out) + rowb + (size_t)c * 2) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

int fill_peers(Peers& P, void* const* bufs, int rank, int world, const char* who) {
  ST_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "%s: rank %d of %d (2..%d ranks)", who, rank,
             world, MAX_RANKS);
  ST_REQUIRE(bufs != nullptr, "%s: null buffer table", who);
  for (int p = 0; p < MAX_RANKS; ++p) P.buf[p] = nullptr;
  for (int p = 0; p < world; ++p) {
    ST_REQUIRE(bufs[p] != nullptr, "%s: buffer of rank %d missing", who, p);
    P.buf[p] = (uint8_t*)bufs[p];
  }
  return 0;
}
}  // namespace

long long st::comm_wait_ns() { return g_wait_ns; }

extern "C" int64_t st_comm_bytes(void) { return (int64_t)COMM_BYTES; }

extern "C" int st_comm_set_timeout_ms(int64_t ms) {
  ST_REQUIRE(ms >= 1 && ms <= 3600000, "st_comm_set_timeout_ms: 1 ms .. 1 h");
  g_wait_ns = ms * 1000000ll;
  return 0;
}

extern "C" int st_comm_alloc(void** buf) {
  ST_REQUIRE(buf != nullptr, "st_comm_alloc: null pointer");
  if (int e = st::cuda_fail(cudaMalloc(buf, COMM_BYTES), "st_comm_alloc")) return e;
  if (int e = st::cuda_fail(cudaMemset(*buf, 0, OFF_RECV), "st_comm_alloc: clear")) return e;
  return st::cuda_fail(cudaMemset((uint8_t*)*buf + OFF_RECV, 0xFF, RECV_BYTES), "st_comm_alloc: clear");
}

extern "C" int st_comm_free(void* buf) { return st::cuda_fail(cudaFree(buf), "st_comm_free"); }

extern "C" int st_comm_export(void* buf, void* handle64) {
  ST_REQUIRE(buf && handle64, "st_comm_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (int e = st::cuda_fail(cudaIpcGetMemHandle(&h, buf), "st_comm_export")) return e;
  memcpy(handle64, &h, 64);
  return 0;
}

extern "C" int st_comm_import(const void* handle64, void** buf) {
  ST_REQUIRE(buf && handle64, "st_comm_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return st::cuda_fail(cudaIpcOpenMemHandle(buf, h, cudaIpcMemLazyEnablePeerAccess), "st_comm_import");
}

extern "C" int st_comm_close(void* buf) { return st::cuda_fail(cudaIpcCloseMemHandle(buf), "st_comm_close"); }

extern "C" int st_allreduce(void* const* bufs, int rank, int world, const void* in, void* out, int64_t n, void* stream) {
  Peers P;
  if (int e = fill_peers(P, bufs, rank, world, "st_allreduce")) return e;
  ST_REQUIRE(n > 0 && n % 8 == 0 && n * 2 <= MAX_BYTES, "st_allreduce: n must be a multiple of 8, at most %lld values",
             (long long)(MAX_BYTES / 2));
  ST_REQUIRE(in && out && st::aligned16(in) && st::aligned16(out), "st_allreduce: null or unaligned pointer");
  int* status = st::status_ptr();
  ST_REQUIRE(status != nullptr, "st_allreduce: no device status word");
  const long long vecs = n / 8;
  long long ctas = (vecs + 255) / 256;                                 // 4 KB per CTA and pass, at most SLOT_BYTES per CTA
  if (ctas > 16) ctas = 16;
  while (((vecs + ctas - 1) / ctas) * 16 > SLOT_BYTES) ++ctas;
  return st::launch("st_allreduce launch", allreduce_kernel, dim3((unsigned)ctas), dim3(256), 0, (cudaStream_t)stream, P,
                    rank, world, (const uint16_t*)in, (uint16_t*)out, (long long)n, status, g_wait_ns);
}

extern "C" int st_allreduce_add_rmsnorm(void* const* bufs, int rank, int world, void* x, const void* delta, const void* w,
                                        void* out, int64_t rows, int64_t cols, double eps, void* stream) {
  Peers P;
  if (int e = fill_peers(P, bufs, rank, world, "st_allreduce_add_rmsnorm")) return e;
  ST_REQUIRE(rows >= 1 && rows <= MAX_CTAS && cols > 0 && cols % 8 == 0 && cols <= 8192,
             "st_allreduce_add_rmsnorm: at most %d rows of at most 8192 columns (a multiple of 8)", MAX_CTAS);
  ST_REQUIRE(x && delta && w && out && st::aligned16(x) && st::aligned16(delta) && st::aligned16(w) && st::aligned16(out),
             "st_allreduce_add_rmsnorm: null or unaligned pointer");
  int* status = st::status_ptr();
  ST_REQUIRE(status != nullptr, "st_allreduce_add_rmsnorm: no device status word");
  return st::launch("st_allreduce_add_rmsnorm launch", allreduce_add_rmsnorm_kernel, dim3((unsigned)rows), dim3(512), 0,
                    (cudaStream_t)stream, P, rank, world, (uint16_t*)x, (const uint16_t*)delta, (const uint16_t*)w,
                    (uint16_t*)out, (int)cols, (float)eps, status, g_wait_ns);
}

// Error text, device properties and the device status word of the statetree_b200 C ABI.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/statetree_b200.h"
#include "st_host.h"

#include <stdlib.h>

namespace {
thread_local char g_err[512] = "";
__device__ int g_status[8];
constexpr int MAX_DEV = 64;
int g_sms[MAX_DEV];
int* g_status_ptr[MAX_DEV];
std::mutex g_mu;
}  // namespace

namespace st {
int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return 1;
}
int cuda_fail(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  return fail("%s: %s", what, cudaGetErrorString(e));
}
bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("STATETREE_PDL");
    on = (v && v[0] == '0') ? 0 : 1;
  }
  return on == 1;
}
int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 148;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}
int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}
}  // namespace st

extern "C" int st_abi_version(void) { return ST_ABI_VERSION; }
extern "C" const char* st_last_error(void) { return g_err; }
extern "C" int st_device_status(void) {
  int h[8] = {0};
  int* p = st::status_ptr();
  if (p == nullptr) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpy(h, p, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return -3;
  if (h[0] != 0) cudaMemset(p, 0, sizeof(h));
  return h[0];
}

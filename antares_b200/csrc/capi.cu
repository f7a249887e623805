// Error reporting and device probe of the antares_b200 C ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace ab200 {

static thread_local char g_err[512] = "";

// Device-side status word: kernels with bounded waits store a site code here when a wait runs out.
__device__ int g_kernel_error = 0;

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_err[0] = 0; }

int *kernel_error_ptr() {
  static int *cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_error) != cudaSuccess) return nullptr;
    cached[dev] = reinterpret_cast<int *>(p);
  }
  return cached[dev];
}

static int g_pdl = 1;  // 0 off, 1 dependents released at kernel start, 2 GEMVs release them after their streaming loop
bool pdl_enabled() { return g_pdl != 0; }
int pdl_mode() { return g_pdl; }
void pdl_set(int mode) { g_pdl = mode; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace ab200

using namespace ab200;

extern "C" const char *ab200_last_error(void) { return g_err; }
extern "C" int ab200_abi_version(void) { return 1; }

extern "C" int ab200_device_info(int device, int *out8_host) {
  clear_error();
  AB200_REQUIRE(out8_host != nullptr, "device_info: null output");
  const cudaDeviceAttr attrs[8] = {cudaDevAttrMultiProcessorCount, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                   cudaDevAttrL2CacheSize, cudaDevAttrClockRate, cudaDevAttrMemoryClockRate,
                                   cudaDevAttrGlobalMemoryBusWidth, cudaDevAttrComputeCapabilityMajor,
                                   cudaDevAttrMaxThreadsPerBlock};
  for (int i = 0; i < 8; ++i) AB200_CUDA(cudaDeviceGetAttribute(&out8_host[i], attrs[i], device));
  int minor = 0;
  AB200_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  out8_host[6] = out8_host[6] * 10 + minor;
  return AB200_OK;
}

extern "C" int ab200_kernel_status(int *status_host) {
  clear_error();
  AB200_REQUIRE(status_host != nullptr, "kernel_status: null output");
  AB200_CUDA(cudaMemcpyFromSymbol(status_host, g_kernel_error, sizeof(int)));
  if (*status_host != 0) {
    const int zero = 0;
    AB200_CUDA(cudaMemcpyToSymbol(g_kernel_error, &zero, sizeof(int)));
    return fail(AB200_ETIMEOUT, "a bounded wait ran out in a kernel (site %d)", *status_host);
  }
  return AB200_OK;
}

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

static void *g_lib_buf[LIB_BUF_COUNT][64] = {};
static size_t g_lib_buf_bytes[LIB_BUF_COUNT][64] = {};
int library_buffer(int which, size_t bytes, size_t min_bytes, size_t zero_bytes, void **out) {
  int dev = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || which < 0 || which >= LIB_BUF_COUNT) return fail(AB200_EUNSUPPORTED, "device index %d out of range", dev);
  void *&buf = g_lib_buf[which][dev];
  size_t &have = g_lib_buf_bytes[which][dev];
  if (have < bytes) {
    const size_t want = bytes < min_bytes ? min_bytes : bytes;
    if (buf) {
      AB200_CUDA(cudaDeviceSynchronize());
      AB200_CUDA(cudaFree(buf));
      buf = nullptr;
      have = 0;
    }
    AB200_CUDA(cudaMalloc(&buf, want));
    if (zero_bytes) AB200_CUDA(cudaMemset(buf, 0, zero_bytes < want ? zero_bytes : want));
    AB200_CUDA(cudaDeviceSynchronize());
    have = want;
  }
  *out = buf;
  return AB200_OK;
}

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

// ---- device memory, copies and timing for hosts that do not link the CUDA runtime themselves ----------
// (the `c-b200` HAL header include/c-b200/backend.hpp maps the reference's `namespace ab` onto these)

extern "C" int ab200_hal_set_device(int device) {
  clear_error();
  AB200_CUDA(cudaSetDevice(device));
  return AB200_OK;
}

extern "C" int ab200_hal_malloc(void **ptr_out_host, size_t bytes) {
  clear_error();
  AB200_REQUIRE(ptr_out_host != nullptr, "hal_malloc: null output");
  AB200_CUDA(cudaMalloc(ptr_out_host, bytes));
  return AB200_OK;
}

extern "C" int ab200_hal_free(void *ptr) {
  clear_error();
  AB200_CUDA(cudaFree(ptr));
  return AB200_OK;
}

extern "C" int ab200_hal_memcpy(void *dst, const void *src, size_t bytes, int kind, void *stream) {
  clear_error();
  AB200_REQUIRE(kind >= 0 && kind <= 2, "hal_memcpy: kind %d (0 host->device, 1 device->host, 2 device->device)", kind);
  const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  AB200_CUDA(cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream));
  return AB200_OK;
}

extern "C" int ab200_hal_synchronize(void *stream) {
  clear_error();
  AB200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return AB200_OK;
}

extern "C" int ab200_hal_event_record(void **event_out_host, void *stream) {
  clear_error();
  AB200_REQUIRE(event_out_host != nullptr, "hal_event_record: null output");
  cudaEvent_t ev;
  AB200_CUDA(cudaEventCreate(&ev));
  AB200_CUDA(cudaEventRecord(ev, (cudaStream_t)stream));
  *event_out_host = ev;
  return AB200_OK;
}

extern "C" int ab200_hal_event_elapsed(void *start_event, void *stop_event, double *seconds_host) {
  clear_error();
  AB200_REQUIRE(start_event && stop_event && seconds_host, "hal_event_elapsed: null argument");
  AB200_CUDA(cudaEventSynchronize((cudaEvent_t)stop_event));
  float ms = 0.f;
  AB200_CUDA(cudaEventElapsedTime(&ms, (cudaEvent_t)start_event, (cudaEvent_t)stop_event));
  AB200_CUDA(cudaEventDestroy((cudaEvent_t)start_event));
  AB200_CUDA(cudaEventDestroy((cudaEvent_t)stop_event));
  *seconds_host = ms * 1e-3;
  return AB200_OK;
}

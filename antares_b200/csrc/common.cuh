// Shared helpers for the antares_b200 kernel library (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/antares_b200.h"

namespace ab200 {

// Records the calling thread's last error text; returns `code` so call sites can `return fail(...)`.
int fail(int code, const char *fmt, ...);
void clear_error();

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks the launch itself (not completion: nothing here synchronises).
#define AB200_CHECK_LAUNCH(what)                                                        \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess) return ::ab200::fail(AB200_ECUDA, "%s: %s", what, cudaGetErrorString(e__)); \
  } while (0)

#define AB200_CUDA(call)                                                                \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess) return ::ab200::fail(AB200_ECUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

#define AB200_REQUIRE(cond, ...)                                                        \
  do {                                                                                  \
    if (!(cond)) return ::ab200::fail(AB200_EINVAL, __VA_ARGS__);                       \
  } while (0)

int sm_count();  // SMs of the current device (cached per device)
void *tensor_map_encoder();  // cuTensorMapEncodeTiled through the runtime's driver entry point query, or nullptr
int *kernel_error_ptr();  // device address of the status word that ab200_kernel_status reads (nullptr on failure)
// Library-owned device buffers, one per user and device: at least `bytes` long (never shorter than min_bytes),
// the first zero_bytes of it zeroed whenever it is allocated or grown (which also synchronises the device).
// Callers keep what they need zero between launches themselves.  Not for use under stream capture before
// the first call; two kernels that use the same buffer must not overlap on the GPU.
enum { LIB_BUF_PERSIST = 0, LIB_BUF_SLABS, LIB_BUF_TC, LIB_BUF_GEMM, LIB_BUF_COUNT };
int library_buffer(int which, size_t bytes, size_t min_bytes, size_t zero_bytes, void **out);

// Programmatic dependent launch: when enabled (option "pdl"), kernels are launched with
// cudaLaunchAttributeProgrammaticStreamSerialization, so a kernel's preamble (weight prefetch)
// overlaps the tail of the kernel before it; every kernel executes griddepcontrol.wait before
// touching data an earlier kernel produced.
void comm_set_wait_polls(unsigned polls);
unsigned comm_wait_polls();
bool pdl_enabled();
int pdl_mode();
void pdl_set(int mode);

// Launch helper: <<<grid, block, smem, stream>>> plus the PDL attribute when enabled.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Paged KV cache: logical cache row s lives in physical row table[s >> shift] * 2^shift + (s mod 2^shift);
// table == nullptr means the cache is contiguous (physical row = s).
struct KvPages {
  const int32_t *table;
  int shift;
};
__device__ __forceinline__ size_t kv_row(const KvPages &pg, int s) {
  return pg.table ? ((size_t)pg.table[s >> pg.shift] << pg.shift) + (size_t)(s & ((1 << pg.shift) - 1)) : (size_t)s;
}

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Split cluster barrier.  A CTA may store into a peer CTA's shared memory only once that peer is
// known to be running: every CTA arrives at kernel start (relaxed: it orders no memory, so it costs
// nothing on the streaming path) and waits just before its first remote store.  Both must be executed by every thread of every CTA of
// the cluster, convergently.
__device__ __forceinline__ void cluster_arrive_started() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_started() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// ---- device helpers ---------------------------------------------------------------------

__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint2 ldg_nc_v2(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

template <int IMM>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(IMM));
  return r;
}

__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace ab200

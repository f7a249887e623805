// One-shot push all-reduce over NVLink peer memory, fused with the decode step's residual update.
//
// The tensor-parallel decode step needs sum all-reduce of a [dim] fp32 partial twice per layer
// (16 KiB at dim 4096): pure latency.  The reference has only NCCL calls inside a TensorFlow op
// (frameworks/tensorflow/communicate_ops.cc:191); here one kernel per rank does the whole
// exchange with plain peer stores and loads - no multicast objects, no TMA, no library call:
//   1. every rank stores its partial into slot `rank` of a receive buffer in EACH rank's own
//      memory (peer stores through NVLink; its own copy is a local store);
//   2. system-scope fence, then it publishes the epoch number in flag `rank` of each rank;
//   3. it waits, with a bounded number of polls, until all flags in its OWN buffer carry the epoch;
//   4. it adds the `world` slots in rank order (every rank gets bit-identical sums) and applies
//      x += fp16_round(sum), the residual update of samples/05_llama2_7b_int4.py:168,173.
// Two slot sets alternate by epoch parity: a rank can only be one all-reduce ahead of the
// slowest rank (it needs that rank's flag to finish), so the set it overwrites has been read.
// A wait that runs out stores a site code in the status word (ab200_kernel_status) and the kernel
// finishes with whatever arrived: the context stays usable and the host sees the error.
#include <cooperative_groups.h>

#include "common.cuh"

namespace ab200 {

constexpr int COMM_MAX_WORLD = 8;
constexpr int COMM_THREADS = 1024;
static unsigned g_comm_wait_polls = 1u << 24;  // polls before a wait gives up (option "comm_wait_polls"); seconds at most

// Receive buffer layout (per rank, in that rank's memory), n_max floats per slot:
//   float slots[2][world][n_max];  int flags[2][COMM_MAX_WORLD];  int epoch;
struct CommPeers {
  float *slots[COMM_MAX_WORLD];  // base of each rank's receive buffer (own entry = local memory)
  int *flags[COMM_MAX_WORLD];
  int *epoch;                    // this rank's epoch counter
  int *status;                   // device status word (ab200_kernel_status)
  int rank, world, n_max;
  unsigned wait_polls;
};

__device__ __forceinline__ void st_release_sys(int *p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int *p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void allreduce_residual_body(const CommPeers &c, float *x, const float *partial, int n) {
  __shared__ int sh_fail;
  const int e = *c.epoch + 1, buf = e & 1;
  if (threadIdx.x == 0) sh_fail = 0;
  // 1. push my partial into slot `rank` of every rank's buffer
  for (int i = threadIdx.x * 4; i < n; i += COMM_THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4 *>(partial + i);
    for (int p = 0; p < c.world; ++p)
      *reinterpret_cast<float4 *>(c.slots[p] + ((size_t)buf * c.world + c.rank) * c.n_max + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish, 3. wait (one thread per peer)
  if (threadIdx.x < c.world) {
    st_release_sys(c.flags[threadIdx.x] + buf * COMM_MAX_WORLD + c.rank, e);
    const int *mine = c.flags[c.rank] + buf * COMM_MAX_WORLD + threadIdx.x;
    unsigned polls = 0;
    while (ld_acquire_sys(mine) < e) {
      if (++polls >= c.wait_polls) {
        atomicExch(c.status, 100 + (int)threadIdx.x);  // site 100 + peer that never arrived
        sh_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  // 4. sum in rank order, residual update
  const float *mine = c.slots[c.rank] + (size_t)buf * c.world * c.n_max;
  for (int i = threadIdx.x * 4; i < n; i += COMM_THREADS * 4) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < c.world; ++p) {
      float4 v;  // L2 only: the slots are written by peers, an L1 line from two epochs ago would be stale
      asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mine + (size_t)p * c.n_max + i) : "memory");
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    float4 r = *reinterpret_cast<float4 *>(x + i);
    r.x += __half2float(__float2half_rn(s.x));
    r.y += __half2float(__float2half_rn(s.y));
    r.z += __half2float(__float2half_rn(s.z));
    r.w += __half2float(__float2half_rn(s.w));
    *reinterpret_cast<float4 *>(x + i) = r;
  }
  __syncthreads();
  if (threadIdx.x == 0) *c.epoch = e;
}

__global__ void __launch_bounds__(COMM_THREADS) allreduce_residual_kernel(CommPeers c, float *x, const float *partial, int n) {
  pdl_launch_dependents();
  pdl_wait();
  allreduce_residual_body(c, x, partial, n);
}

// All ranks in one launch on one GPU (rank = blockIdx.x): the protocol check for machines with
// fewer GPUs than ranks.  Blocks wait on one another, so the launch is cooperative.
struct CommEmu {
  CommPeers peers[COMM_MAX_WORLD];
  float *x[COMM_MAX_WORLD];
  const float *partial[COMM_MAX_WORLD];
};
__global__ void __launch_bounds__(COMM_THREADS) allreduce_residual_emulated_kernel(const CommEmu *emu, int n) {
  const CommPeers c = emu->peers[blockIdx.x];
  allreduce_residual_body(c, emu->x[blockIdx.x], emu->partial[blockIdx.x], n);
}

static size_t comm_bytes(int world, int n_max) {
  return (size_t)2 * world * n_max * sizeof(float) + (size_t)(2 * COMM_MAX_WORLD + 4) * sizeof(int);
}

static void fill_peers(CommPeers &c, void *const *bufs, int rank, int world, int n_max) {
  c.status = kernel_error_ptr();
  c.wait_polls = g_comm_wait_polls;
  for (int p = 0; p < world; ++p) {
    c.slots[p] = reinterpret_cast<float *>(bufs[p]);
    c.flags[p] = reinterpret_cast<int *>(reinterpret_cast<char *>(bufs[p]) + (size_t)2 * world * n_max * sizeof(float));
  }
  c.epoch = c.flags[rank] + 2 * COMM_MAX_WORLD;
  c.rank = rank;
  c.world = world;
  c.n_max = n_max;
}

void comm_set_wait_polls(unsigned v) { g_comm_wait_polls = v; }

}  // namespace ab200

using namespace ab200;

extern "C" size_t ab200_comm_buffer_bytes(int world, int n_max) { return comm_bytes(world, n_max); }

extern "C" int ab200_comm_alloc(int world, int n_max, void **buf_out, void *ipc_handle64_host) {
  clear_error();
  AB200_REQUIRE(buf_out && world >= 1 && world <= COMM_MAX_WORLD && n_max > 0 && n_max % 4 == 0, "comm_alloc: bad argument (world 1..8, n_max a multiple of 4)");
  const size_t bytes = comm_bytes(world, n_max);
  AB200_CUDA(cudaMalloc(buf_out, bytes));
  AB200_CUDA(cudaMemset(*buf_out, 0, bytes));
  AB200_CUDA(cudaDeviceSynchronize());
  if (ipc_handle64_host) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    AB200_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(ipc_handle64_host), *buf_out));
  }
  return AB200_OK;
}

extern "C" int ab200_comm_open(const void *ipc_handle64_host, void **peer_buf_out) {
  clear_error();
  AB200_REQUIRE(ipc_handle64_host && peer_buf_out, "comm_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle64_host, sizeof(h));
  AB200_CUDA(cudaIpcOpenMemHandle(peer_buf_out, h, cudaIpcMemLazyEnablePeerAccess));
  return AB200_OK;
}

extern "C" int ab200_comm_close(void *peer_buf) {
  clear_error();
  AB200_CUDA(cudaIpcCloseMemHandle(peer_buf));
  return AB200_OK;
}

extern "C" int ab200_comm_free(void *buf) {
  clear_error();
  AB200_CUDA(cudaFree(buf));
  return AB200_OK;
}

extern "C" int ab200_allreduce_residual(float *x_f32, const float *partial_f32, int n, void *const *bufs_host, int rank, int world,
                                        int n_max, void *stream) {
  clear_error();
  AB200_REQUIRE(x_f32 && partial_f32 && bufs_host, "allreduce_residual: null pointer");
  AB200_REQUIRE(world >= 1 && world <= COMM_MAX_WORLD && rank >= 0 && rank < world, "allreduce_residual: rank %d / world %d", rank, world);
  AB200_REQUIRE(n > 0 && n % 4 == 0 && n <= n_max, "allreduce_residual: n=%d must be a multiple of 4, at most n_max=%d", n, n_max);
  AB200_REQUIRE(aligned16(x_f32) && aligned16(partial_f32), "allreduce_residual: pointers must be 16-byte aligned");
  CommPeers c{};
  fill_peers(c, bufs_host, rank, world, n_max);
  AB200_CUDA(launch_pdl(allreduce_residual_kernel, dim3(1), dim3(COMM_THREADS), 0, (cudaStream_t)stream, c, x_f32, partial_f32, n));
  return AB200_OK;
}

extern "C" int ab200_allreduce_residual_emulated(float *const *x_host, const float *const *partial_host, int n, void *const *bufs_host,
                                                 int world, int n_max, void *emu_scratch_dev, void *stream) {
  clear_error();
  AB200_REQUIRE(x_host && partial_host && bufs_host && emu_scratch_dev, "allreduce_residual_emulated: null pointer");
  AB200_REQUIRE(world >= 1 && world <= COMM_MAX_WORLD && n > 0 && n % 4 == 0 && n <= n_max, "allreduce_residual_emulated: bad sizes");
  CommEmu emu{};
  for (int r = 0; r < world; ++r) {
    fill_peers(emu.peers[r], bufs_host, r, world, n_max);
    emu.x[r] = x_host[r];
    emu.partial[r] = partial_host[r];
  }
  AB200_CUDA(cudaMemcpyAsync(emu_scratch_dev, &emu, sizeof(emu), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  AB200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));  // `emu` is a stack object
  const CommEmu *dev_emu = reinterpret_cast<const CommEmu *>(emu_scratch_dev);
  void *args[] = {(void *)&dev_emu, (void *)&n};
  AB200_CUDA(cudaLaunchCooperativeKernel((void *)allreduce_residual_emulated_kernel, dim3(world), dim3(COMM_THREADS), args, 0, (cudaStream_t)stream));
  return AB200_OK;
}

extern "C" size_t ab200_comm_emulation_scratch_bytes(void) { return sizeof(CommEmu); }

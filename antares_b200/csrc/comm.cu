// One-shot push all-reduce over NVLink peer memory, fused with the decode step's residual update.
//
// The tensor-parallel decode step needs sum all-reduce of a [dim] fp32 partial twice per layer
// (16 KiB at dim 4096): pure latency.  The reference has only NCCL calls inside a TensorFlow op
// (frameworks/tensorflow/communicate_ops.cc:191); here one kernel per rank does the whole
// exchange with plain peer stores and local loads - no multicast objects, no TMA, no library call -
// and the data carries its own arrival flag, so a value crosses NVLink exactly once and nothing
// waits for a store to be acknowledged:
//   1. every rank stores each element of its partial as the 8-byte pair (value, epoch) into slot
//      `rank` of a receive buffer in EACH peer's memory (two pairs per 16-byte store; an aligned
//      8-byte pair arrives whole or not at all);
//   2. it polls, with a bounded number of polls, the pairs its peers store into its OWN buffer
//      until their epoch field carries this exchange's number;
//   3. it adds the `world` contributions in rank order (every rank gets bit-identical sums; its
//      own contribution comes straight from `partial`) and applies x += fp16_round(sum), the
//      residual update of samples/05_llama2_7b_int4.py:168,173.
// Two slot sets alternate by epoch parity: a rank can only be one all-reduce ahead of the
// slowest rank (it needs that rank's data to finish), so the set it overwrites has been read.
// A wait that runs out stores a site code in the status word (ab200_kernel_status) and the kernel
// finishes with whatever arrived: the context stays usable and the host sees the error.
#include <cooperative_groups.h>
#include <math_constants.h>

#include "common.cuh"

namespace ab200 {

constexpr int COMM_MAX_WORLD = 8;
constexpr int COMM_THREADS = 1024;
static unsigned g_comm_wait_polls = 1u << 24;  // polls before a wait gives up (option "comm_wait_polls"); seconds at most

// Receive buffer layout (per rank, in that rank's memory), n_max (value, epoch) pairs per slot:
//   uint2 slots[2][world][n_max];  int epoch;  int ticket (used by the all-reduce fused into the
//   row-parallel GEMV, w4a16_gemv_ring.cu);
struct CommPeers {
  uint2 *slots[COMM_MAX_WORLD];  // base of each rank's receive buffer (own entry = local memory)
  int *epoch;                    // this rank's epoch counter
  int *status;                   // device status word (ab200_kernel_status)
  int rank, world, n_max;
  unsigned wait_polls;
};

__device__ __forceinline__ void allreduce_residual_body(const CommPeers &c, float *x, const float *partial, int n) {
  const int e = *c.epoch + 1, buf = e & 1;
  const unsigned tag = (unsigned)e;
  // A wait that ran out earlier stays in the status word until the host reads it: every later
  // exchange then skips its polls at once instead of spinning to its own limit again (one dead
  // peer must not hold the GPU for 64 limits per token).
  bool failed = *reinterpret_cast<volatile int *>(c.status) != 0;
  for (int i = threadIdx.x * 4; i < n; i += COMM_THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4 *>(partial + i);
    // 1. push (value, epoch) pairs into slot `rank` of every peer's buffer
    const uint4 lo = make_uint4(__float_as_uint(v.x), tag, __float_as_uint(v.y), tag);
    const uint4 hi = make_uint4(__float_as_uint(v.z), tag, __float_as_uint(v.w), tag);
    for (int p = 0; p < c.world; ++p) {
      if (p == c.rank) continue;
      uint2 *dst = c.slots[p] + ((size_t)buf * c.world + c.rank) * c.n_max + i;
      asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
      asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 2), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
    }
  }
  // 2. collect the peers' pairs from my own buffer, 3. sum in rank order, residual update
  for (int i = threadIdx.x * 4; i < n; i += COMM_THREADS * 4) {
    const float4 mine = *reinterpret_cast<const float4 *>(partial + i);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < c.world; ++p) {
      float4 v = mine;
      if (p != c.rank) {
        const uint2 *src = c.slots[c.rank] + ((size_t)buf * c.world + p) * c.n_max + i;
        uint4 lo, hi;
        unsigned polls = 0;
        for (;;) {
          asm volatile("ld.relaxed.sys.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "l"(src) : "memory");
          asm volatile("ld.relaxed.sys.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(src + 2) : "memory");
          if ((lo.y == tag) & (lo.w == tag) & (hi.y == tag) & (hi.w == tag)) break;
          if (failed || ++polls >= c.wait_polls) {
            if (!failed) atomicExch(c.status, 100 + p);  // site 100 + peer that never arrived
            failed = true;                               // give up on everything still missing
            break;
          }
        }
        v = make_float4(__uint_as_float(lo.x), __uint_as_float(lo.z), __uint_as_float(hi.x), __uint_as_float(hi.z));
      }
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

// Vocabulary-parallel greedy step: every rank takes the argmax of its own logits shard, the
// (value, global index) pairs are exchanged with the same flag-in-data pushes as above (two 8-byte
// pairs per rank), every rank picks the same winner (highest value, lowest index on ties, like
// torch.argmax over the gathered logits) and does the loop bookkeeping of the single-GPU
// greedy_next kernel.  Replaces the logits all-gather + argmax of the classifier step.
__device__ __forceinline__ void greedy_next_tp_body(const CommPeers &c, const float *__restrict__ logits, int n, int vocab_offset,
                                                    const int32_t *__restrict__ prompt, int n_prompt, int32_t *token_dev, int32_t *pos_dev,
                                                    int32_t *out_tokens, int out_cap) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int sh_fail;
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  const int nvec = ((reinterpret_cast<uintptr_t>(logits) & 15u) == 0) ? n / 4 : 0;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += COMM_THREADS) {
    const float4 v = reinterpret_cast<const float4 *>(logits)[i0];
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e[j] > best || (e[j] == best && i0 * 4 + j < bi)) { best = e[j]; bi = i0 * 4 + j; }
  }
  for (int i = nvec * 4 + threadIdx.x; i < n; i += COMM_THREADS) {
    const float v = logits[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  if (threadIdx.x == 0) sh_fail = 0;
  __syncthreads();
  if (warp != 0) return;
  best = sv[lane];
  bi = si[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  // every lane of warp 0 now holds this rank's winner; lane p talks to peer p
  const int gi = (bi == 0x7fffffff) ? 0x7fffffff : bi + vocab_offset;
  const int e = *c.epoch + 1, buf = e & 1;
  const unsigned tag = (unsigned)e;
  float pv = -CUDART_INF_F;
  int pi = 0x7fffffff;
  if (lane < c.world) {
    if (lane == c.rank) {
      pv = best;
      pi = gi;
    } else {
      uint2 *dst = c.slots[lane] + ((size_t)buf * c.world + c.rank) * c.n_max;
      asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(__float_as_uint(best)), "r"(tag), "r"((unsigned)gi), "r"(tag) : "memory");
      const uint2 *src = c.slots[c.rank] + ((size_t)buf * c.world + lane) * c.n_max;
      uint4 w;
      unsigned polls = (*reinterpret_cast<volatile int *>(c.status) != 0) ? c.wait_polls - 1 : 0;  // an earlier timeout is sticky: one poll only
      for (;;) {
        asm volatile("ld.relaxed.sys.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
        if ((w.y == tag) & (w.w == tag)) break;
        if (++polls >= c.wait_polls) {
          atomicExch(c.status, 120 + lane);  // site 120 + peer whose candidate never arrived
          sh_fail = 1;
          break;
        }
      }
      pv = __uint_as_float(w.x);
      pi = (int)w.z;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, pv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, pi, o);
    if (ov > pv || (ov == pv && oi < pi)) { pv = ov; pi = oi; }
  }
  if (lane == 0) {
    const int pos = *pos_dev;
    int next = (pi == 0x7fffffff) ? 0 : pi;
    if (prompt != nullptr && pos + 1 < n_prompt) next = prompt[pos + 1];
    *token_dev = next;
    if (out_tokens == nullptr) {
      *pos_dev = pos + 1;
    } else if (pos + 1 < out_cap) {  // past the end of the token log: nothing is stored, the position stays put
      out_tokens[pos + 1] = next;
      *pos_dev = pos + 1;
    }
    *c.epoch = e;
  }
}

__global__ void __launch_bounds__(COMM_THREADS) greedy_next_tp_kernel(CommPeers c, const float *__restrict__ logits, int n, int vocab_offset,
                                                                      const int32_t *__restrict__ prompt, int n_prompt, int32_t *token_dev,
                                                                      int32_t *pos_dev, int32_t *out_tokens, int out_cap) {
  pdl_launch_dependents();
  pdl_wait();
  greedy_next_tp_body(c, logits, n, vocab_offset, prompt, n_prompt, token_dev, pos_dev, out_tokens, out_cap);
}

// All ranks of the greedy exchange as the blocks of one cooperative launch (single-GPU protocol check).
struct GreedyEmu {
  CommPeers peers[COMM_MAX_WORLD];
  const float *logits[COMM_MAX_WORLD];
  int n[COMM_MAX_WORLD], offset[COMM_MAX_WORLD];
  int32_t *token[COMM_MAX_WORLD], *pos[COMM_MAX_WORLD], *out_tokens[COMM_MAX_WORLD];
  int out_cap;
};
__global__ void __launch_bounds__(COMM_THREADS) greedy_next_tp_emulated_kernel(const GreedyEmu *emu, const int32_t *prompt, int n_prompt) {
  const int r = blockIdx.x;
  const CommPeers c = emu->peers[r];
  greedy_next_tp_body(c, emu->logits[r], emu->n[r], emu->offset[r], prompt, n_prompt, emu->token[r], emu->pos[r], emu->out_tokens[r], emu->out_cap);
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
  return (size_t)2 * world * n_max * sizeof(uint2) + 4 * sizeof(int);
}

static void fill_peers(CommPeers &c, void *const *bufs, int rank, int world, int n_max) {
  c.status = kernel_error_ptr();
  c.wait_polls = g_comm_wait_polls;
  for (int p = 0; p < world; ++p) c.slots[p] = reinterpret_cast<uint2 *>(bufs[p]);
  c.epoch = reinterpret_cast<int *>(reinterpret_cast<char *>(bufs[rank]) + (size_t)2 * world * n_max * sizeof(uint2));
  c.rank = rank;
  c.world = world;
  c.n_max = n_max;
}

void comm_set_wait_polls(unsigned v) { g_comm_wait_polls = v; }
unsigned comm_wait_polls() { return g_comm_wait_polls; }

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

extern "C" size_t ab200_comm_emulation_scratch_bytes(void) { return sizeof(CommEmu) > sizeof(GreedyEmu) ? sizeof(CommEmu) : sizeof(GreedyEmu); }

extern "C" int ab200_greedy_next_tp_emulated(const float *const *logits_host, const int *n_local_host, const int *offset_host, void *const *bufs_host,
                                             int world, int n_max, const int32_t *prompt, int n_prompt, int32_t *const *token_host,
                                             int32_t *const *pos_host, int32_t *const *out_tokens_host, int out_cap, void *emu_scratch_dev,
                                             void *stream) {
  clear_error();
  AB200_REQUIRE(logits_host && n_local_host && offset_host && bufs_host && token_host && pos_host && out_tokens_host && emu_scratch_dev,
                "greedy_next_tp_emulated: null pointer");
  AB200_REQUIRE(world >= 1 && world <= COMM_MAX_WORLD && n_max >= 4 && n_max % 4 == 0, "greedy_next_tp_emulated: bad sizes");
  GreedyEmu emu{};
  emu.out_cap = out_cap;
  for (int r = 0; r < world; ++r) {
    fill_peers(emu.peers[r], bufs_host, r, world, n_max);
    emu.logits[r] = logits_host[r];
    emu.n[r] = n_local_host[r];
    emu.offset[r] = offset_host[r];
    emu.token[r] = token_host[r];
    emu.pos[r] = pos_host[r];
    emu.out_tokens[r] = out_tokens_host[r];
  }
  AB200_CUDA(cudaMemcpyAsync(emu_scratch_dev, &emu, sizeof(emu), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  AB200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));  // `emu` is a stack object
  const GreedyEmu *dev_emu = reinterpret_cast<const GreedyEmu *>(emu_scratch_dev);
  void *args[] = {(void *)&dev_emu, (void *)&prompt, (void *)&n_prompt};
  AB200_CUDA(cudaLaunchCooperativeKernel((void *)greedy_next_tp_emulated_kernel, dim3(world), dim3(COMM_THREADS), args, 0, (cudaStream_t)stream));
  return AB200_OK;
}

extern "C" int ab200_greedy_next_tp(const float *logits_local_f32, int n_local, int vocab_offset, void *const *bufs_host, int rank, int world,
                                    int n_max, const int32_t *prompt, int n_prompt, int32_t *token_dev, int32_t *pos_dev,
                                    int32_t *out_tokens, int out_cap, void *stream) {
  clear_error();
  AB200_REQUIRE(logits_local_f32 && bufs_host && token_dev && pos_dev && n_local > 0 && vocab_offset >= 0, "greedy_next_tp: bad argument");
  AB200_REQUIRE(world >= 1 && world <= COMM_MAX_WORLD && rank >= 0 && rank < world, "greedy_next_tp: rank %d / world %d", rank, world);
  AB200_REQUIRE(n_max >= 4 && n_max % 4 == 0, "greedy_next_tp: the exchange buffer must hold at least 4 pairs per slot");
  CommPeers c{};
  fill_peers(c, bufs_host, rank, world, n_max);
  AB200_CUDA(launch_pdl(greedy_next_tp_kernel, dim3(1), dim3(COMM_THREADS), 0, (cudaStream_t)stream, c, logits_local_f32, n_local, vocab_offset,
                        prompt, n_prompt, token_dev, pos_dev, out_tokens, out_cap));
  return AB200_OK;
}

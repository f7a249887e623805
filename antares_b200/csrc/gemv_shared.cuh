// Pieces shared by the two W4A16 decode GEMV kernels (scalar-pipe and warp-MMA).
#pragma once
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"

namespace ab200 {

constexpr int TILE_N = 128;   // columns per CTA: 32 lanes x 4
constexpr int UNIT_ROWS = 4;  // packed rows per work unit
constexpr int UNIT_K = UNIT_ROWS * 8;

// Epilogues: fp16 store; fp32 residual += fp16-rounded result; fp32 store (tensor-parallel partials).
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_STORE_F32 = 2 };

// (q-8) for the eight nibbles of `w` as four half2: (n0,n4) (n1,n5) (n2,n6) (n3,n7).
// 0x6400 | q is the fp16 number 1024+q; the high nibble of each byte gives 1024+16q, brought
// back with one HFMA2 (x/16 - 72), so only one shift is needed per word.
__device__ __forceinline__ void unpack8(uint32_t w, __half2 (&v)[4]) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u, MAGIC = 0x64006400u;
  const __half2 c1032 = u2h2(0x64086408u);  // (1032, 1032)
  const __half2 c16th = u2h2(0x2C002C00u);  // (1/16, 1/16)
  const __half2 cm72 = u2h2(0xD480D480u);   // (-72, -72)
  const uint32_t w8 = w >> 8;
  const uint32_t t0 = lop3<0xEA>(w, LO, MAGIC);  // (a & b) | c
  const uint32_t t1 = lop3<0xEA>(w, HI, MAGIC);
  const uint32_t t2 = lop3<0xEA>(w8, LO, MAGIC);
  const uint32_t t3 = lop3<0xEA>(w8, HI, MAGIC);
  v[0] = __hsub2(u2h2(t0), c1032);
  v[1] = __hfma2(u2h2(t1), c16th, cm72);
  v[2] = __hsub2(u2h2(t2), c1032);
  v[3] = __hfma2(u2h2(t3), c16th, cm72);
}

__device__ __forceinline__ void mma16816p(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  // not volatile: a pure function of its operands, so the compiler may schedule loads around it
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float4 ldcg_f4(const float *p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 permute_row(uint4 v) {  // (x0..x7) -> (x0,x4)(x1,x5)(x2,x6)(x3,x7)
  uint4 o;
  o.x = __byte_perm(v.x, v.z, 0x5410);
  o.y = __byte_perm(v.x, v.z, 0x7632);
  o.z = __byte_perm(v.y, v.w, 0x5410);
  o.w = __byte_perm(v.y, v.w, 0x7632);
  return o;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// A-operand quad for two MMAs from two packed words (columns c and c+1 of this thread):
// lo = {(k0,k4) of w0, (k0,k4) of w1, (k1,k5) of w0, (k1,k5) of w1}, hi = same for (k2,k6)/(k3,k7).
__device__ __forceinline__ void unpack_pair(uint32_t w0, uint32_t w1, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u, MAGIC = 0x64006400u;
  const __half2 c1032 = u2h2(0x64086408u), c16th = u2h2(0x2C002C00u), cm72 = u2h2(0xD480D480u);
  const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
  lo[0] = h22u(__hsub2(u2h2(lop3<0xEA>(w0, LO, MAGIC)), c1032));
  lo[1] = h22u(__hsub2(u2h2(lop3<0xEA>(w1, LO, MAGIC)), c1032));
  lo[2] = h22u(__hfma2(u2h2(lop3<0xEA>(w0, HI, MAGIC)), c16th, cm72));
  lo[3] = h22u(__hfma2(u2h2(lop3<0xEA>(w1, HI, MAGIC)), c16th, cm72));
  hi[0] = h22u(__hsub2(u2h2(lop3<0xEA>(w0s, LO, MAGIC)), c1032));
  hi[1] = h22u(__hsub2(u2h2(lop3<0xEA>(w1s, LO, MAGIC)), c1032));
  hi[2] = h22u(__hfma2(u2h2(lop3<0xEA>(w0s, HI, MAGIC)), c16th, cm72));
  hi[3] = h22u(__hfma2(u2h2(lop3<0xEA>(w1s, HI, MAGIC)), c16th, cm72));
}

// The same operand quads as raw fp16 bit patterns: a nibble q left in mantissa bits 0-3 is the
// subnormal q * 2^-24, in bits 4-7 it is 16q * 2^-24.  No FP16-pipe instruction at all; the
// caller divides the matching x values by 16 for the high nibbles, removes the zero-point
// through -8 * sum(x), and rescales the fp32 sums by 2^24.
__device__ __forceinline__ void unpack_pair_raw(uint32_t w0, uint32_t w1, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
  const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
  lo[0] = w0 & LO;
  lo[1] = w1 & LO;
  lo[2] = w0 & HI;
  lo[3] = w1 & HI;
  hi[0] = w0s & LO;
  hi[1] = w1s & LO;
  hi[2] = w0s & HI;
  hi[3] = w1s & HI;
}

// Cross-warp, then cross-CTA (cluster) reduction of per-thread fp32 partials, and the epilogue.
// Warps 0..NWARPS-1 hold partials (facc[m][c] for columns lane*4+c); every thread of the CTA
// must call this (it contains CTA and cluster barriers).  The order of every sum is fixed, so
// results are bitwise repeatable.  red: [NWARPS][M][128] floats; part: M * 128 floats used as an
// inbox [source rank][M][128 / cluster size].
//
// Push model: every CTA adds its warps' partials per column and STORES the sum into the inbox of
// the CTA that owns the column (rank r owns columns [r * 128/cs, (r+1) * 128/cs)); one cluster
// barrier later each owner adds the cs entries of its inbox in rank order and writes the result.
// Remote stores do not wait for a round trip and nothing reads a peer's memory after the
// barrier, so no second barrier is needed before exit.  The caller's kernel must have executed
// cluster_arrive_started() at its top (when the cluster has more than one CTA): the matching wait
// here proves that every peer CTA is running before its shared memory is written.
template <int M, int EPI, int NTHREADS, int NWARPS>
__device__ __forceinline__ void reduce_and_store(float (&facc)[M][4], float *red, float *part, void *out, int N, int tile_n0) {
  namespace cg = cooperative_groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp < NWARPS) {
#pragma unroll
    for (int m = 0; m < M; ++m)
      *reinterpret_cast<float4 *>(&red[(warp * M + m) * TILE_N + lane * 4]) = make_float4(facc[m][0], facc[m][1], facc[m][2], facc[m][3]);
  }
  __syncthreads();
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), rank = cluster.block_rank();
  const int cols_per = TILE_N / cs;  // cs in {1,2,4,8}
  if (cs > 1) cluster_wait_started();
  for (int i = threadIdx.x; i < M * TILE_N; i += NTHREADS) {
    const int m = i / TILE_N, c = i % TILE_N;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) s += red[(w * M + m) * TILE_N + c];
    const int owner = c / cols_per, cc = c - owner * cols_per;
    float *inbox = (cs > 1) ? cluster.map_shared_rank(part, owner) : part;
    inbox[(rank * M + m) * cols_per + cc] = s;
  }
  if (cs > 1) cluster.sync(); else __syncthreads();
  for (int i = threadIdx.x; i < M * cols_per; i += NTHREADS) {
    const int m = i / cols_per, cc = i - m * cols_per;
    float s = 0.f;
    for (unsigned r = 0; r < cs; ++r) s += part[(r * M + m) * cols_per + cc];
    const int n = tile_n0 + rank * cols_per + cc;
    if (n < N) {
      if (EPI == EPI_STORE) {
        reinterpret_cast<__half *>(out)[(size_t)m * N + n] = __float2half_rn(s);
      } else if (EPI == EPI_STORE_F32) {
        reinterpret_cast<float *>(out)[(size_t)m * N + n] = s;
      } else {
        float *o = reinterpret_cast<float *>(out) + (size_t)m * N + n;
        *o += __half2float(__float2half_rn(s));
      }
    }
  }
}

// warp-MMA variant (w4a16_gemv_mma.cu)
bool gemv_mma_eligible(int dtype, int M, int K, int N);
int gemv_mma_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                      int K, int N, int group, int epi, cudaStream_t s);
int gemv_tuning_set(const char *name, int value);
int gemv_tuning_impl();

// TMA-ring variant (w4a16_gemv_tma.cu)
bool gemv_tma_eligible(int dtype, int M, int K, int N, int group);
int gemv_tma_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                      int K, int N, int group, int epi, cudaStream_t s, bool *handled);

// TMA ring with the activations streamed through it (w4a16_gemv_slab.cu): batch 5-16
bool gemv_slab_eligible(int dtype, int M, int K, int N, int group);
size_t gemv_slab_scratch_bytes(int M, int K);
int gemv_slab_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                       int K, int N, int group, int epi, void *scratch, cudaStream_t s, bool *handled);

// tcgen05 variant, weights as the A operand in tensor memory (w4a16_gemv_tc.cu): batch 1-16
bool gemv_tc_eligible(int dtype, int M, int K, int N, int group);
int gemv_tc_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M, int K,
                     int N, int group, int epi, cudaStream_t s, bool *handled);

// persistent balanced variant (w4a16_gemv_persist.cu)
enum { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_SILU_MUL = 2 };
constexpr size_t PERSIST_COUNTER_BYTES = 64 * 1024;  // counters live at the start of the scratch: up to 16384 column tiles
size_t gemv_persist_scratch_bytes(int M, int K, int N);
bool gemv_persist_fits(int M, int K, int N);
int gemv_persist_dispatch(const void *x, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                          int K, int N, int group, int pro, int epi, void *scratch, cudaStream_t s);
int gemv_tuning_cluster();

// bulk-copy ring variant (w4a16_gemv_ring.cu): batch 1, group 128, N % 128 == 0; `tiled` selects the
// tile-major weight layout (linear bulk copies) or the reference layout (tensor-map copies)
bool gemv_ring_eligible(int M, int K, int N, int group, bool tiled);
int gemv_ring_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int K, int N,
                       int epi, bool tiled, cudaStream_t s, void *const *comm_bufs = nullptr, int rank = 0, int world = 1, int n_max = 0);
int gemv_ring_set_depth(int d);

}  // namespace ab200

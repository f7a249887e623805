// W4A16 decode GEMV, warp-MMA variant (fp16 activations/scales), batch 1..16.
//
// Why this exists: the scalar-pipe variant (w4a16_gemv.cu) spends ~3 lane-instructions per
// nibble, and on sm_100 both the integer/logic pipe and the FP16 pipe issue at half rate, so it
// saturates instruction issue at ~45% of HBM bandwidth.  Here the multiply-accumulate of every
// dequantised nibble goes through `mma.sync.m16n8k16` (fp16 x fp16 -> fp32): the scalar pipes
// only unpack (1 SHF + 4 LOP3 per word) and remove the zero-point (4 HSUB2/HFMA2 per word),
// independent of the batch size.  The weights are the A operand (16 output columns x 16 k),
// the activations the B operand (16 k x 8 batch rows); batch rows beyond M are zero.
//
// Data path: unchanged HBM layout (qweight int32 [K/8, N]).  A warp owns 32 columns; lane
// (g = lane/4, t = lane%4) loads the 16-byte chunk g (4 columns) of packed row 4s+t, so one warp
// copy instruction reads 4 rows x 128 contiguous bytes.  The stream is `cp.async` (16 B, L2-only)
// into a per-warp shared-memory ring MMA_DEPTH units deep (10 KiB of weights in flight per warp,
// 160 KiB per SM at two CTAs), each lane reading back only what it copied.  Because the four lanes of an MMA
// "thread group" hold different packed rows, one MMA contracts 16 k-values taken from 4 packed
// rows x the nibble pairs (k0,k4)(k1,k5) [or (k2,k6)(k3,k7)] that the 0x6400 unpack produces; x is
// staged in shared memory in the same order.  MMA accumulators hold un-scaled sums of one
// quantisation group; they are folded into fp32 running sums with the group scale.
// CTA = 128 columns (4 column warps) x 2 K warps; the K slices of a column tile form a cluster and
// meet in distributed shared memory in fixed order (deterministic; no scratch, no atomics).
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int MMA_WN = 4;  // column warps: 4 x 32 columns = TILE_N
constexpr int MMA_WK = 2;  // K warps
constexpr int MMA_THREADS = MMA_WN * MMA_WK * 32;
constexpr int UNIT_STEPS = 4;               // steps (4 packed rows = 32 k) per unit
constexpr int UNIT128 = UNIT_STEPS * UNIT_K;  // 128 k per unit
constexpr int XS_PAD = 32;                  // halves: batch rows 64 B apart modulo 128 B -> conflict-free LDS.128
constexpr int MMA_DEPTH_DEFAULT = 5;        // units (2 KiB of weights each) in flight per warp
constexpr int SLOT_BYTES = UNIT_STEPS * 512 + 4 * 256;  // weights [4 steps][32 lanes][16 B] + scales [<=4][32 lanes][8 B]

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async8(void *dst, const void *src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct MmaGemvParams {
  const __half *x;
  const int32_t *qw;
  const __half *scales;
  void *out;
  int M, K, N, group;
  int units;      // ceil(K / 128)
  int xs_stride;  // halves between batch rows of x in shared memory; the same in every CTA of a
                  // cluster, so that `part` sits at one offset cluster-wide
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MB = 8 (batch <= 8) or 16.  SPG = steps per scale group inside a unit: 4 (group % 128 == 0), 2 (group 64), 1 (group 32).
template <int MB, int SPG, int EPI, int MMA_DEPTH>
__global__ void __launch_bounds__(MMA_THREADS) w4a16_gemv_mma_kernel(MmaGemvParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int NB = MB / 8;  // B-fragment sets
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wn = warp % MMA_WN, wk = warp / MMA_WN;
  const int g = lane >> 2, t = lane & 3;
  const int tile_n0 = tile * TILE_N;
  const int n0 = tile_n0 + wn * 32 + g * 4;  // this thread's 4 columns
  const bool col_ok = n0 < p.N;
  const int M = p.M;

  const int ub = (int)((long)p.units * krank / cs), ue = (int)((long)p.units * (krank + 1) / cs);
  const int k_begin = ub * UNIT128;
  const int k_end = (ue * UNIT128 < p.K) ? ue * UNIT128 : p.K;
  const int kslice = (k_end > k_begin) ? (k_end - k_begin) : 0;  // multiple of 32
  const int xs_stride = p.xs_stride;

  __half *xs = reinterpret_cast<__half *>(smem_raw);
  float *red = reinterpret_cast<float *>(smem_raw + (((size_t)M * xs_stride * 2 + 15) & ~(size_t)15));  // [WK][M][128]
  float *part = red + MMA_WK * M * TILE_N;                                                              // [M][128]

  const int rows_total = kslice / 8;
  const int total_rows_K = p.K / 8;
  const int32_t *qbase = p.qw + n0;
  const __half *sbase = p.scales + n0;

  // Per-warp ring of DEPTH units in shared memory, filled with cp.async.  Every lane copies
  // exactly the 16-byte chunks it will itself read back (slot layout [step][lane] -> LDS.128 is
  // conflict-free), so completion is tracked per thread with cp.async groups and no barrier.
  unsigned char *wring = reinterpret_cast<unsigned char *>(part + M * TILE_N) + (size_t)warp * MMA_DEPTH * SLOT_BYTES;
  auto issue_unit = [&](int u, int slot) {
    unsigned char *dst = wring + (size_t)slot * SLOT_BYTES;
#pragma unroll
    for (int s = 0; s < UNIT_STEPS; ++s) {
      const int row = u * (UNIT128 / 8) + s * 4 + t;
      const bool ok = col_ok && row < total_rows_K;
      cp_async16(dst + (s * 32 + lane) * 16, ok ? (const void *)(qbase + (size_t)row * p.N) : (const void *)p.qw, ok ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < UNIT_STEPS / SPG; ++i) {
      const int k = u * UNIT128 + i * SPG * UNIT_K;
      const bool ok = col_ok && k < p.K;
      cp_async8(dst + UNIT_STEPS * 512 + (i * 32 + lane) * 8, ok ? (const void *)(sbase + (size_t)(k / p.group) * p.N) : (const void *)p.scales, ok ? 8 : 0);
    }
  };

  const int n_my = (ue - ub - wk + MMA_WK - 1) / MMA_WK;  // units this warp owns: ub+wk, ub+wk+WK, ...
#pragma unroll
  for (int i = 0; i < MMA_DEPTH; ++i) {
    if (i < n_my) issue_unit(ub + wk + i * MMA_WK, i);
    cp_async_commit();
  }

  // Stage x: per packed row the 8 values are stored as (x0,x4)(x1,x5)(x2,x6)(x3,x7).
  for (int i = threadIdx.x; i < M * rows_total; i += MMA_THREADS) {
    const int m = i / rows_total, r = i % rows_total;
    const uint4 v = *reinterpret_cast<const uint4 *>(p.x + (size_t)m * p.K + k_begin + r * 8);
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = o;
  }
  __syncthreads();

  float facc[NB][2][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) facc[nb][j][i] = 0.f;

  for (int iu = 0; iu < n_my; ++iu) {
    cp_async_wait<MMA_DEPTH - 1>();  // this thread's copies of unit iu have landed
    const int uu = ub + wk + iu * MMA_WK;
    const int slot = iu % MMA_DEPTH;
    const unsigned char *src = wring + (size_t)slot * SLOT_BYTES;
    float d[NB][2][4];
#pragma unroll
    for (int s = 0; s < UNIT_STEPS; ++s) {
      if (s % SPG == 0) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) d[nb][j][i] = 0.f;
      }
      const int r_local = (uu - ub) * (UNIT128 / 8) + s * 4 + t;  // packed row relative to the CTA slice
      uint4 xb[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const int m = g + nb * 8;
        if (m < M && r_local < rows_total) xb[nb] = *reinterpret_cast<const uint4 *>(xs + (size_t)m * xs_stride + r_local * 8);
        else xb[nb] = make_uint4(0, 0, 0, 0);
      }
      const uint4 wv = *reinterpret_cast<const uint4 *>(src + (s * 32 + lane) * 16);
      const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        __half2 v0[4], v1[4];
        unpack8(wr[2 * j], v0);
        unpack8(wr[2 * j + 1], v1);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma16816(d[nb][j], h22u(v0[0]), h22u(v1[0]), h22u(v0[1]), h22u(v1[1]), xb[nb].x, xb[nb].y);
          mma16816(d[nb][j], h22u(v0[2]), h22u(v1[2]), h22u(v0[3]), h22u(v1[3]), xb[nb].z, xb[nb].w);
        }
      }
      if (s % SPG == SPG - 1) {
        const uint2 sv = *reinterpret_cast<const uint2 *>(src + UNIT_STEPS * 512 + ((s / SPG) * 32 + lane) * 8);
        const float2 s01 = __half22float2(u2h2(sv.x)), s23 = __half22float2(u2h2(sv.y));
        const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            facc[nb][j][0] = fmaf(sc[2 * j], d[nb][j][0], facc[nb][j][0]);
            facc[nb][j][1] = fmaf(sc[2 * j], d[nb][j][1], facc[nb][j][1]);
            facc[nb][j][2] = fmaf(sc[2 * j + 1], d[nb][j][2], facc[nb][j][2]);
            facc[nb][j][3] = fmaf(sc[2 * j + 1], d[nb][j][3], facc[nb][j][3]);
          }
      }
    }
    // Refill the slot just drained (same thread wrote and read it: program order suffices).
    if (iu + MMA_DEPTH < n_my) issue_unit(uu + MMA_DEPTH * MMA_WK, slot);
    cp_async_commit();
  }
  cp_async_wait<0>();

  // ---- reduction: K warps -> CTA partial -> cluster (fixed order) -> epilogue ------------------
  // facc[nb][j][i]: column wn*32 + g*4 + 2j + (i>>1), batch nb*8 + 2t + (i&1).
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = nb * 8 + 2 * t + (i & 1);
        if (m < M) red[(wk * M + m) * TILE_N + wn * 32 + g * 4 + 2 * j + (i >> 1)] = facc[nb][j][i];
      }
  __syncthreads();
  for (int i = threadIdx.x; i < M * TILE_N; i += MMA_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < MMA_WK; ++w) s += red[w * M * TILE_N + i];
    part[i] = s;
  }
  if (cs > 1) cluster.sync(); else __syncthreads();
  const int cols_per = TILE_N / cs;
  for (int i = threadIdx.x; i < M * cols_per; i += MMA_THREADS) {
    const int m = i / cols_per, c = krank * cols_per + i % cols_per;
    float s = 0.f;
    for (unsigned r = 0; r < cs; ++r) {
      const float *remote = (cs > 1) ? cluster.map_shared_rank(part, r) : part;
      s += remote[m * TILE_N + c];
    }
    const int n = tile_n0 + c;
    if (n < p.N) {
      if (EPI == EPI_STORE) reinterpret_cast<__half *>(p.out)[(size_t)m * p.N + n] = __float2half_rn(s);
      else if (EPI == EPI_STORE_F32) reinterpret_cast<float *>(p.out)[(size_t)m * p.N + n] = s;
      else reinterpret_cast<float *>(p.out)[(size_t)m * p.N + n] += __half2float(__float2half_rn(s));
    }
  }
  if (cs > 1) cluster.sync();
}

// ---- host side -------------------------------------------------------------------------------

struct GemvTuning {
  int cluster = 0;  // 0 = heuristic
  int impl = 0;     // 0 = auto (MMA), 1 = scalar pipes, 2 = MMA
  int depth = 0;    // 0 = default ring depth
};
static GemvTuning g_tune;

static int pick_cluster_mma(int tiles, int units) {
  if (g_tune.cluster > 0) return g_tune.cluster;
  const int target = 2 * sm_count();
  int cs = 1;
  while (cs < 8 && tiles * cs < target && units / (cs * 2) >= MMA_WK) cs *= 2;
  return cs;
}

template <typename Kern>
static int launch_mma(Kern kern, MmaGemvParams p, int depth, cudaStream_t stream) {
  const size_t RING_BYTES = (size_t)MMA_WN * MMA_WK * depth * SLOT_BYTES;
  const int tiles = (p.N + TILE_N - 1) / TILE_N;
  int cs = pick_cluster_mma(tiles, p.units);
  auto smem_for = [&](int c) {
    const int units_max = (p.units + c - 1) / c;
    return (((size_t)p.M * (units_max * UNIT128 + XS_PAD) * 2 + 15) & ~(size_t)15) + (size_t)(MMA_WK + 1) * p.M * TILE_N * sizeof(float) + RING_BYTES;
  };
  while (smem_for(cs) > 200 * 1024 && cs < 8) cs *= 2;
  const size_t smem = smem_for(cs);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: K=%d x M=%d does not fit shared memory", p.K, p.M);
  p.xs_stride = ((p.units + cs - 1) / cs) * UNIT128 + XS_PAD;
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * cs, 1, 1);
  cfg.blockDim = dim3(MMA_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return AB200_OK;
}

bool gemv_mma_eligible(int dtype, int M) { return dtype == AB200_F16 && g_tune.impl != 1; }

template <int MB, int EPI>
static int mma_by_group(const MmaGemvParams &p, cudaStream_t s) {
  constexpr int D = MMA_DEPTH_DEFAULT;
  if (p.group % 128 == 0) {
    switch (g_tune.depth) {
      case 2: return launch_mma(w4a16_gemv_mma_kernel<MB, 4, EPI, 2>, p, 2, s);
      case 3: return launch_mma(w4a16_gemv_mma_kernel<MB, 4, EPI, 3>, p, 3, s);
      case 4: return launch_mma(w4a16_gemv_mma_kernel<MB, 4, EPI, 4>, p, 4, s);
      case 6: return launch_mma(w4a16_gemv_mma_kernel<MB, 4, EPI, 6>, p, 6, s);
      default: return launch_mma(w4a16_gemv_mma_kernel<MB, 4, EPI, D>, p, D, s);
    }
  }
  if (p.group % 64 == 0) return launch_mma(w4a16_gemv_mma_kernel<MB, 2, EPI, D>, p, D, s);
  return launch_mma(w4a16_gemv_mma_kernel<MB, 1, EPI, D>, p, D, s);
}

template <int EPI>
static int mma_by_batch(const MmaGemvParams &p, cudaStream_t s) {
  return (p.M <= 8) ? mma_by_group<8, EPI>(p, s) : mma_by_group<16, EPI>(p, s);
}

int gemv_mma_dispatch(const void *x, const int32_t *qw, const void *scales, void *out, int M, int K, int N, int group, int epi,
                      cudaStream_t s) {
  MmaGemvParams p{reinterpret_cast<const __half *>(x), qw, reinterpret_cast<const __half *>(scales), out, M, K, N, group,
                  (K + UNIT128 - 1) / UNIT128, 0};
  if (epi == EPI_STORE) return mma_by_batch<EPI_STORE>(p, s);
  if (epi == EPI_RESIDUAL) return mma_by_batch<EPI_RESIDUAL>(p, s);
  return mma_by_batch<EPI_STORE_F32>(p, s);
}

int gemv_tuning_set(const char *name, int value) {
  if (!strcmp(name, "gemv_cluster")) {
    if (!(value == 0 || value == 1 || value == 2 || value == 4 || value == 8)) return fail(AB200_EINVAL, "gemv_cluster must be 0, 1, 2, 4 or 8");
    g_tune.cluster = value;
  } else if (!strcmp(name, "pdl")) {
    pdl_set(value != 0);
  } else if (!strcmp(name, "gemv_depth")) {
    if (value != 0 && (value < 2 || value > 6)) return fail(AB200_EINVAL, "gemv_depth must be 0 or 2..6");
    g_tune.depth = value;
  } else if (!strcmp(name, "gemv_impl")) {
    if (value < 0 || value > 3) return fail(AB200_EINVAL, "gemv_impl must be 0 (auto), 1 (scalar pipes), 2 (cluster warp MMA) or 3 (persistent warp MMA)");
    g_tune.impl = value;
  } else {
    return fail(AB200_EINVAL, "unknown option %s", name);
  }
  return AB200_OK;
}

int gemv_tuning_cluster() { return g_tune.cluster; }
int gemv_tuning_impl() { return g_tune.impl; }

}  // namespace ab200

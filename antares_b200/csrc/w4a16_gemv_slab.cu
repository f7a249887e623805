// W4A16 decode GEMV for batches of 5-16 rows (fp16, group 128): TMA ring for the weights AND for the
// activations, raw-nibble warp-MMA consumers.
//
// Replaces the kernel the reference generates from samples/05_llama2_7b_int4.py:135-139 when it is called
// with 5..16 batch rows.
//
// The TMA-ring kernel for small batches (w4a16_gemv_tma.cu) keeps a CTA's whole K slice of the
// activations in shared memory; at 8-16 rows that is 33-66 KiB per CTA, which leaves room for a ring of two
// stages only, and its warps then wait on the stage barriers.  Here the activations travel through the ring
// with the weights: a small kernel first writes them once, in the order and scaling the MMA B operand wants,
// as one contiguous "slab" per 256-k stage
//     slab(S) = [MB rows][256 k + 32 pad] fp16, packed row r of batch row m holding (x0,x4)(x1,x5)/16 (x2,x6)(x3,x7)/16,
//               then [2 groups][MB] fp32 accumulator seeds  -8 * 2^-24 * sum over the group of x
// (rows past M and k past K are zeros), and the GEMV's producer thread brings slab S into the stage with one
// linear bulk copy next to the stage's four weight boxes and two scale rows.  Shared memory then holds
// nothing but the ring (21-26 KiB per stage), the staging prologues (plain / RMSNorm / SiLU*up) live in
// the small kernel, and the consumer loop is the one of the small-batch kernel reading its B operands from
// the stage instead of from a resident copy.  Every CTA re-reads the slabs of its K slice from L2 (25 MB
// for the widest projection at 16 rows).
//
// Programmatic dependent launch: the slab kernel releases its dependents at once and waits for its own
// inputs; the GEMV issues the weight and scale copies of its first ring fill before griddepcontrol.wait and
// the slab copies after it (the slabs are what the kernel before it writes).  Split-K over a cluster with
// the push reduction of the other GEMV kernels; every mbarrier wait bounded (status sites 500/510).
#include <cooperative_groups.h>
#include <cuda.h>  // CUtensorMap (types only)

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int S_CWARPS = 8;                        // consumer warps: 4 column groups x 2 K halves
constexpr int S_WN = 4;
constexpr int S_THREADS = (S_CWARPS + 1) * 32;     // + the producer warp
constexpr int S_STAGE_K = 256;                     // k per stage = 32 packed rows = 2 groups of 128
constexpr int S_BOX_BYTES = 32 * 128;              // one weight box: 32 packed rows x 32 columns x 4 B
constexpr int S_W_BYTES = 4 * S_BOX_BYTES;         // 16 KiB of packed weights per stage
constexpr int S_SC_BYTES = 2 * TILE_N * 2;         // two scale rows x 128 columns, fp16
constexpr int S_XROW = S_STAGE_K + 32;             // halves per batch row of a slab: rows 64 B apart modulo 128 B
constexpr int S_MAX_DEPTH = 8;

__host__ __device__ constexpr int slab_bytes(int MB) { return MB * S_XROW * 2 + 2 * MB * 4; }

struct SlabPrepParams {
  const void *x;
  const __half *norm_w;
  unsigned char *slabs;
  int M, MB, K, stages;
  float eps;
};

// One CTA per batch row (rows M..MB-1: zero rows).  Thread = packed rows tid, tid + 256, ...
template <int PRO>
__global__ void __launch_bounds__(256) gemv_slab_prep_kernel(SlabPrepParams p) {
  __shared__ float sh[8];
  pdl_launch_dependents();
  pdl_wait();  // the activations come from the kernel before; the slabs may still be read by the GEMV before that one
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int K = p.K, rows_total = p.stages * 32, rows_valid = K / 8, sb = slab_bytes(p.MB);
  float rs = 1.f;
  if (PRO == PRO_RMSNORM && m < p.M) {
    const float *xg = reinterpret_cast<const float *>(p.x) + (size_t)m * K;
    float ss = 0.f;
    for (int r = threadIdx.x; r < rows_valid; r += 256) {
      const float4 a = *reinterpret_cast<const float4 *>(xg + r * 8), b = *reinterpret_cast<const float4 *>(xg + r * 8 + 4);
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) sh[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += sh[w];
    rs = rsqrtf(tot * (1.0f / (float)K) + p.eps);
  }
  for (int r0 = 0; r0 < rows_total; r0 += 256) {  // whole warps: the group sums below use shuffles
    const int r = r0 + threadIdx.x;
    const bool inside = m < p.M && r < rows_valid;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (inside) {
      if (PRO == PRO_PLAIN) {
        o = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(p.x) + (size_t)m * K + r * 8);
      } else if (PRO == PRO_SILU_MUL) {
        const __half *xg = reinterpret_cast<const __half *>(p.x) + (size_t)m * 2 * K;
        const uint4 gv = *reinterpret_cast<const uint4 *>(xg + r * 8), uv = *reinterpret_cast<const uint4 *>(xg + K + r * 8);
        const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
          q[j] = h22u(__floats2half2_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y));
        }
        o = make_uint4(q[0], q[1], q[2], q[3]);
      } else {
        const float *xr = reinterpret_cast<const float *>(p.x) + (size_t)m * K + r * 8;
        const float4 a = *reinterpret_cast<const float4 *>(xr), b = *reinterpret_cast<const float4 *>(xr + 4);
        const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + r * 8);
        const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)), w3 = __half22float2(u2h2(wv.w));
        o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
        o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
        o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
        o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
      }
    }
    const float2 f0 = __half22float2(u2h2(o.x)), f1 = __half22float2(u2h2(o.y)), f2 = __half22float2(u2h2(o.z)), f3 = __half22float2(u2h2(o.w));
    float sx = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) sx += __shfl_xor_sync(0xffffffffu, sx, off);  // 16 packed rows = one group
    if (r < rows_total) {
      uint4 q = permute_row(o);
      const __half2 c16th = u2h2(0x2C002C00u);
      q.y = h22u(__hmul2(u2h2(q.y), c16th));
      q.w = h22u(__hmul2(u2h2(q.w), c16th));
      unsigned char *slab = p.slabs + (size_t)(r / 32) * sb;
      *reinterpret_cast<uint4 *>(slab + ((size_t)m * S_XROW + (r % 32) * 8) * 2) = q;
      if (r % 16 == 0) reinterpret_cast<float *>(slab + (size_t)p.MB * S_XROW * 2)[((r % 32) / 16) * p.MB + m] = sx * (-8.0f * 5.9604644775390625e-8f);
    }
  }
}

struct SlabGemvParams {
  const unsigned char *slabs;
  void *out;
  int *status;
  int M, K, N;
  int stages;  // ceil(K / 256)
  int depth;   // ring stages
  unsigned wait_polls;
};

__device__ __forceinline__ uint32_t s_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool s_mbar_wait(uint32_t bar, unsigned parity, unsigned polls) {
  {  // non-blocking probe first: cheaper than try_wait when the phase has already completed
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  for (unsigned i = 0; i < polls; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void s_tma_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void s_bulk(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}

// MB = 8 (batch <= 8) or 16.
template <int MB, int EPI>
__global__ void __launch_bounds__(S_THREADS, 3) w4a16_gemv_slab_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                                                                     SlabGemvParams p) {
  extern __shared__ unsigned char s_smem[];
  __shared__ __align__(8) unsigned long long sh_bars[2 * S_MAX_DEPTH];
  constexpr int NB = MB / 8;
  constexpr int SLAB = slab_bytes(MB);
  constexpr int STAGE = S_W_BYTES + S_SC_BYTES + SLAB;  // weights (1024-aligned) | scales | slab; a multiple of 128
  constexpr int STAGE_PAD = (STAGE + 1023) & ~1023;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile_n0 = tile * TILE_N;
  const int M = p.M, N = p.N, D = p.depth;
  const int st_begin = (int)((long)p.stages * krank / cs), st_end = (int)((long)p.stages * (krank + 1) / cs);
  const int nst = st_end - st_begin;

  // shared memory: [ring: D stages, 1024-aligned][inbox M x 128 floats]
  const uint32_t base_u32 = s_smem_u32(s_smem);
  const uint32_t ring = (base_u32 + 1023u) & ~1023u;
  unsigned char *ring_p = s_smem + (ring - base_u32);
  float *red = reinterpret_cast<float *>(ring_p);  // [2][M][128]: reuses the ring once every consumer has left the K loop
  float *part = reinterpret_cast<float *>(ring_p + (size_t)D * STAGE_PAD);
  const uint32_t bars = s_smem_u32(sh_bars);  // full[D], empty[D]

  if (threadIdx.x == 0) {
    for (int i = 0; i < D; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * (D + i)), "n"(S_CWARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (cs > 1) cluster_arrive_started();
  pdl_launch_dependents();
  __syncthreads();

  if (warp == S_CWARPS) {
    // ---- producer ---------------------------------------------------------------------------------------
    {
      auto issue_weights = [&](int i, int slot) {
        const uint32_t full = bars + 8 * slot, dst = ring + slot * STAGE_PAD;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "n"(STAGE) : "memory");
        const int row = (st_begin + i) * 32;
#pragma unroll
        for (int b = 0; b < 4; ++b) s_tma_2d(dst + b * S_BOX_BYTES, &tm_w, tile_n0 + b * 32, row, full);
        s_tma_2d(dst + S_W_BYTES, &tm_s, tile_n0, (st_begin + i) * 2, full);
      };
      auto issue_slab = [&](int i, int slot) {
        s_bulk(ring + slot * STAGE_PAD + S_W_BYTES + S_SC_BYTES, p.slabs + (size_t)(st_begin + i) * SLAB, SLAB, bars + 8 * slot);
      };
      // first ring fill: weights and scales at once (they never depend on the kernel before), slabs after the wait
      const int first = nst < D ? nst : D;
      if (lane == 0)
        for (int i = 0; i < first; ++i) issue_weights(i, i);
      pdl_wait();  // the whole warp: its threads read a residual output in the epilogue
      if (lane == 0)
        for (int i = 0; i < first; ++i) issue_slab(i, i);
      int slot = 0, round = 1;
      for (int i = first; lane == 0 && i < nst; ++i) {
        if (!s_mbar_wait(bars + 8 * (D + slot), (round - 1) & 1, p.wait_polls)) {
          atomicExch(p.status, 500 + slot);  // site 500: a ring stage was never released
          break;
        }
        issue_weights(i, slot);
        issue_slab(i, slot);
        if (++slot == D) {
          slot = 0;
          ++round;
        }
      }
    }
  } else {
    // ---- consumers ----------------------------------------------------------------------------------------
    const int wn = warp % S_WN, wk = warp / S_WN;
    const int g = lane >> 2, t = lane & 3;
    const int chunk = ((g & 1) << 2) | (g >> 1);  // 16-byte chunk (4 columns) of the warp's 32-column box
    pdl_wait();  // a residual output may come from the kernel before this one
    // per-lane operand offsets inside a stage
    uint32_t x_off[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) x_off[nb] = (uint32_t)(S_W_BYTES + S_SC_BYTES + ((g + nb * 8) * S_XROW) * 2 + wk * 256 + t * 16);
    const uint32_t c_off = (uint32_t)(S_W_BYTES + S_SC_BYTES + MB * S_XROW * 2 + (wk * MB + 2 * t) * 4);
    // weights: packed row wk*16 + 4s + t of box wn; the swizzle XORs the chunk with (row & 7) = 4(s&1) + t
    const uint32_t w_row = (uint32_t)(wn * S_BOX_BYTES + wk * 2048 + t * 128);
    const uint32_t w_off0 = w_row + (uint32_t)((chunk ^ t) << 4), w_off1 = w_row + (uint32_t)((chunk ^ t ^ 4) << 4);
    const uint32_t s_off = (uint32_t)(S_W_BYTES + wk * 256 + (wn * 32 + chunk * 4) * 2);

    float facc[NB][2][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) facc[nb][j][i] = 0.f;

    int slot = 0, round = 0;
    bool alive = true;
    for (int i = 0; i < nst; ++i) {
      if (alive && !s_mbar_wait(bars + 8 * slot, round & 1, p.wait_polls)) {
        if (lane == 0) atomicExch(p.status, 510 + slot);  // site 510: a ring stage never arrived
        alive = false;                                    // stop waiting; the result is void
      }
      const unsigned char *st = ring_p + (size_t)slot * STAGE_PAD;
      float d[NB][2][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const float2 seed = *reinterpret_cast<const float2 *>(st + c_off + nb * 32);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          d[nb][j][0] = d[nb][j][2] = seed.x;
          d[nb][j][1] = d[nb][j][3] = seed.y;
        }
      }
      uint4 wv[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) wv[s] = *reinterpret_cast<const uint4 *>(st + s * 512 + ((s & 1) ? w_off1 : w_off0));
      const uint2 sv = *reinterpret_cast<const uint2 *>(st + s_off);
      // one batch block: all of the stage's operands fit in registers and the slot goes back before the math;
      // two blocks: the activations are read step by step and the slot goes back after the last read
      constexpr int XS = NB == 1 ? 4 : 1;
      uint4 xc[XS][NB];
      if (NB == 1) {
#pragma unroll
        for (int s = 0; s < XS; ++s) xc[s][0] = *reinterpret_cast<const uint4 *>(st + x_off[0] + s * 64);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bars + 8 * (D + slot)) : "memory");
      }
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (NB > 1) {
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) xc[0][nb] = *reinterpret_cast<const uint4 *>(st + x_off[nb] + s * 64);
          if (s == 3) {
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bars + 8 * (D + slot)) : "memory");
          }
        }
        const int xi = NB == 1 ? s : 0;
        const uint32_t wr[4] = {wv[s].x, wv[s].y, wv[s].z, wv[s].w};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t lo[4], hi[4];
          unpack_pair_raw(wr[2 * j], wr[2 * j + 1], lo, hi);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            mma16816p(d[nb][j], lo[0], lo[1], lo[2], lo[3], xc[xi][nb].x, xc[xi][nb].y);
            mma16816p(d[nb][j], hi[0], hi[1], hi[2], hi[3], xc[xi][nb].z, xc[xi][nb].w);
          }
        }
      }
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
      if (++slot == D) {
        slot = 0;
        ++round;
      }
    }

    asm volatile("bar.sync 1, %0;" ::"n"(S_CWARPS * 32) : "memory");  // every consumer is done with the ring: `red` may overwrite it
    // facc[nb][j][i]: column wn*32 + chunk*4 + 2j + (i>>1), batch nb*8 + 2t + (i&1)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = nb * 8 + 2 * t + (i & 1);
          if (m < M) red[(wk * M + m) * TILE_N + wn * 32 + chunk * 4 + 2 * j + (i >> 1)] = facc[nb][j][i] * 16777216.0f;
        }
  }
  __syncthreads();

  // ---- reduction: K halves -> owner CTA's inbox (push) -> one cluster barrier -> rank-ordered sum -> epilogue
  const int cols_per = TILE_N / cs;
  if (cs > 1) cluster_wait_started();  // every peer CTA is running: its inbox may be written
  for (int i = threadIdx.x; i < M * TILE_N; i += S_THREADS) {
    const int m = i / TILE_N, c = i - m * TILE_N;
    const float v = red[i] + red[M * TILE_N + i];
    const int owner = c / cols_per, cc = c - owner * cols_per;
    float *inbox = (cs > 1) ? cluster.map_shared_rank(part, owner) : part;
    inbox[(krank * M + m) * cols_per + cc] = v;
  }
  if (cs > 1) cluster.sync(); else __syncthreads();
  for (int i = threadIdx.x; i < M * cols_per; i += S_THREADS) {
    const int m = i / cols_per, cc = i - m * cols_per;
    float s = 0.f;
    for (unsigned r = 0; r < cs; ++r) s += part[(r * M + m) * cols_per + cc];
    const int n = tile_n0 + krank * cols_per + cc;
    if (n < N) {
      if (EPI == EPI_STORE) reinterpret_cast<__half *>(p.out)[(size_t)m * N + n] = __float2half_rn(s);
      else if (EPI == EPI_STORE_F32) reinterpret_cast<float *>(p.out)[(size_t)m * N + n] = s;
      else reinterpret_cast<float *>(p.out)[(size_t)m * N + n] += __half2float(__float2half_rn(s));
    }
  }
}

// ---- host side -------------------------------------------------------------------------------

typedef CUresult (*SlabEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Library-owned slab buffer (at most 43 stages x 9.2 KiB for the 7B shapes): allocated by the first call that needs it.
static int slab_scratch(size_t bytes, void **out) { return library_buffer(LIB_BUF_SLABS, bytes, (size_t)1 << 20, 0, out); }

bool gemv_slab_eligible(int dtype, int M, int K, int N, int group) {
  return dtype == AB200_F16 && group == 128 && K % 128 == 0 && N % 8 == 0 && M >= 5 && M <= 16 && tensor_map_encoder() != nullptr;
}

template <int MB, int EPI>
static int launch_slab(const CUtensorMap &tm_w, const CUtensorMap &tm_s, const SlabGemvParams &p, int tiles, int cs, size_t smem, cudaStream_t stream) {
  auto kern = w4a16_gemv_slab_kernel<MB, EPI>;
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * cs, 1, 1);
  cfg.blockDim = dim3(S_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_s, p));
  return AB200_OK;
}

template <int MB>
static int slab_by_epi(const CUtensorMap &tm_w, const CUtensorMap &tm_s, const SlabGemvParams &p, int tiles, int cs, size_t smem, int epi, cudaStream_t s) {
  if (epi == EPI_STORE) return launch_slab<MB, EPI_STORE>(tm_w, tm_s, p, tiles, cs, smem, s);
  if (epi == EPI_RESIDUAL) return launch_slab<MB, EPI_RESIDUAL>(tm_w, tm_s, p, tiles, cs, smem, s);
  return launch_slab<MB, EPI_STORE_F32>(tm_w, tm_s, p, tiles, cs, smem, s);
}

// Sets *handled when this variant took the call (see gemv_tma_dispatch for the convention).
size_t gemv_slab_scratch_bytes(int M, int K) { return (size_t)((K + S_STAGE_K - 1) / S_STAGE_K) * slab_bytes(M <= 8 ? 8 : 16); }

// `scratch`: caller's workspace for the slabs (gemv_slab_scratch_bytes), or nullptr for the library-owned buffer.
int gemv_slab_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                       int K, int N, int group, int epi, void *scratch, cudaStream_t s, bool *handled) {
  *handled = false;
  if (!gemv_slab_eligible(AB200_F16, M, K, N, group)) return AB200_OK;
  const int MB = M <= 8 ? 8 : 16;
  const int stages = (K + S_STAGE_K - 1) / S_STAGE_K, tiles = (N + TILE_N - 1) / TILE_N;
  const int slab = slab_bytes(MB), stage_pad = ((S_W_BYTES + S_SC_BYTES + slab) + 1023) & ~1023;
  // K split: enough CTAs for every SM to hold three, every CTA at least two stages
  const int sms = sm_count();
  int cs = gemv_tuning_cluster();
  if (cs <= 0) {
    cs = 1;
    while (cs < 8 && tiles * cs * 2 <= 3 * sms && stages / (cs * 2) >= 2) cs *= 2;
  }
  while (cs > 1 && stages / cs < 1) cs /= 2;
  const int st_max = (stages + cs - 1) / cs;
  int per_sm = (tiles * cs + sms - 1) / sms;
  if (per_sm > 3) per_sm = 3;
  if (per_sm < 1) per_sm = 1;
  const size_t fixed = 1024 + (size_t)M * TILE_N * sizeof(float);
  int depth = (int)(((size_t)225 * 1024 / per_sm - 1024 - fixed) / stage_pad);
  if (depth > st_max) depth = st_max;
  if (depth > S_MAX_DEPTH) depth = S_MAX_DEPTH;
  if (depth < 1) return AB200_OK;
  if ((size_t)depth * stage_pad < (size_t)2 * M * TILE_N * sizeof(float)) return AB200_OK;  // `red` reuses the ring
  const size_t smem = fixed + (size_t)depth * stage_pad;

  void *slabs = scratch;
  if (!slabs) {
    if (int rc = slab_scratch((size_t)stages * slab, &slabs)) return rc;
  }
  SlabEncodeFn enc = reinterpret_cast<SlabEncodeFn>(tensor_map_encoder());
  CUtensorMap tm_w, tm_s;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 8)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    const cuuint32_t box[2] = {32, 32}, estr[2] = {1, 1};
    const CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(qw), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AB200_ECUDA, "w4a16_gemv: cuTensorMapEncodeTiled(qweight) failed with %d", (int)r);
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 128)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {TILE_N, 2}, estr[2] = {1, 1};
    const CUresult r = enc(&tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(scales), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AB200_ECUDA, "w4a16_gemv: cuTensorMapEncodeTiled(scales) failed with %d", (int)r);
  }
  int *status = kernel_error_ptr();
  if (!status) return fail(AB200_ECUDA, "w4a16_gemv: status word unavailable");
  *handled = true;
  SlabPrepParams pp{x, norm_w, reinterpret_cast<unsigned char *>(slabs), M, MB, K, stages, eps};
  cudaError_t e;
  if (pro == PRO_PLAIN) e = launch_pdl(gemv_slab_prep_kernel<PRO_PLAIN>, dim3(MB), dim3(256), 0, s, pp);
  else if (pro == PRO_RMSNORM) e = launch_pdl(gemv_slab_prep_kernel<PRO_RMSNORM>, dim3(MB), dim3(256), 0, s, pp);
  else e = launch_pdl(gemv_slab_prep_kernel<PRO_SILU_MUL>, dim3(MB), dim3(256), 0, s, pp);
  if (e != cudaSuccess) return fail(AB200_ECUDA, "w4a16_gemv (slab kernel): %s", cudaGetErrorString(e));
  SlabGemvParams p{reinterpret_cast<const unsigned char *>(slabs), out, status, M, K, N, stages, depth, 1u << 22};
  return MB == 8 ? slab_by_epi<8>(tm_w, tm_s, p, tiles, cs, smem, epi, s) : slab_by_epi<16>(tm_w, tm_s, p, tiles, cs, smem, epi, s);
}

}  // namespace ab200

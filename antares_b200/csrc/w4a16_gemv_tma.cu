// W4A16 decode GEMV, TMA-ring variant (fp16 activations/scales, group 128, batch 1..16).
//
// The other GEMV kernels fetch weights with per-thread loads, so the bytes a CTA has in flight
// are bounded by registers (or by per-warp cp.async rings) and every warp stalls on its own loads.
// Here one producer thread per CTA keeps a shared-memory ring of DEPTH stages full with tensor-map
// TMA copies (`cp.async.bulk.tensor.2d`, completion on an mbarrier): a stage is 256 k x 128 columns
// of packed weights (four 32-column boxes of 32 packed rows x 128 B, 128-byte swizzle) plus the two
// scale rows of its two quantisation groups.  With 2-3 CTAs per SM that is 130-200 KiB of weights
// in flight per SM regardless of what the consumer warps are doing, and the copies of the first
// DEPTH stages start before the activations exist (they do not depend on the kernel before).
//
// Eight consumer warps (4 column groups x 2 K halves of a stage) read their operands back with
// conflict-free 16-byte loads (the g -> chunk mapping below plus the swizzle puts the eight lanes
// of a quarter warp in eight different bank groups) and contract them on `mma.sync.m16n8k16`
// with the raw-nibble operand trick of w4a16_gemv_mma.cu: the scalar pipes only shift and mask
// (1 SHF + 4 LOP3 per packed word), the zero-point enters as the accumulator seed
// -8 * sum(x) * 2^-24 per group, fp32 sums are scaled by 2^24 at the end.  A consumer warp
// releases a stage with one mbarrier arrive; the producer refills it as soon as all eight have.
//
// Split-K: the stages of a column tile are divided over the CTAs of a thread-block cluster; every
// CTA pushes its column sums into the owner CTA's inbox in distributed shared memory, one cluster
// barrier, rank-ordered sum (bitwise repeatable; no scratch, no atomics, no remote reads).
// Every mbarrier wait is bounded: when one runs out the kernel stores a site code in the status
// word (ab200_kernel_status), stops waiting and finishes with whatever it has.
#include <cooperative_groups.h>
#include <cuda.h>  // CUtensorMap and its enums (types only; the encoder is fetched through the runtime)

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int T_CWARPS = 8;                        // consumer warps: 4 column groups x 2 K halves
constexpr int T_WN = 4;
constexpr int T_THREADS = (T_CWARPS + 1) * 32;     // + the producer warp
constexpr int T_CTHREADS = T_CWARPS * 32;
constexpr int T_STAGE_K = 256;                     // k per stage = 32 packed rows = 2 groups of 128
constexpr int T_BOX_BYTES = 32 * 128;              // one box: 32 packed rows x 32 columns x 4 B
constexpr int T_W_BYTES = 4 * T_BOX_BYTES;         // 16 KiB of packed weights per stage
constexpr int T_S_BYTES = 2 * TILE_N * 2;          // two scale rows x 128 columns, fp16
constexpr int T_XS_PAD = 32;                       // halves: batch rows 64 B apart modulo 128 B
constexpr int T_MAX_DEPTH = 8;

struct TmaGemvParams {
  const void *x;
  const __half *norm_w;
  void *out;
  int *status;
  int M, K, N;
  int stages;     // ceil(K / 256)
  int xs_stride;  // halves between batch rows of x in shared memory (cluster-uniform)
  int depth;      // ring stages
  float eps;
  unsigned wait_polls;
};

__device__ __forceinline__ uint32_t t_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool t_mbar_wait(uint32_t bar, unsigned parity, unsigned polls) {
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

__device__ __forceinline__ void t_tma_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
               : "memory");
}

// MB = 8 (batch <= 8) or 16.
template <int MB, int PRO, int EPI>
__global__ void __launch_bounds__(T_THREADS) w4a16_gemv_tma_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                   const __grid_constant__ CUtensorMap tm_s, TmaGemvParams p) {
  extern __shared__ unsigned char t_smem[];
  __shared__ float sh_ss[T_CWARPS];
  constexpr int NB = MB / 8;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile_n0 = tile * TILE_N;
  const int M = p.M, N = p.N, K = p.K, D = p.depth;

  // this CTA's stages
  const int st_begin = (int)((long)p.stages * krank / cs), st_end = (int)((long)p.stages * (krank + 1) / cs);
  const int nst = st_end - st_begin;
  const int k_begin = st_begin * T_STAGE_K;
  const int xs_stride = p.xs_stride;

  // shared memory: [ring of weights, 1024-aligned][ring of scales][mbarriers][256 B zeros][x][inbox][seeds]
  const uint32_t base_u32 = t_smem_u32(t_smem);
  const uint32_t ring_w = (base_u32 + 1023u) & ~1023u;
  unsigned char *ring_wp = t_smem + (ring_w - base_u32);
  const uint32_t ring_s = ring_w + D * T_W_BYTES;
  unsigned char *ring_sp = ring_wp + D * T_W_BYTES;
  const uint32_t bars = ring_s + D * T_S_BYTES;  // full[D], empty[D]
  unsigned char *misc = ring_sp + D * T_S_BYTES + 256;  // 16 * D <= 128 bytes of barriers, rounded to 256
  __half *xs = reinterpret_cast<__half *>(misc + 256);
  float *red = reinterpret_cast<float *>(ring_wp);  // [2][M][128]: reuses the ring once every consumer has left the K loop
  float *part = reinterpret_cast<float *>(misc + 256 + (((size_t)M * xs_stride * 2 + 15) & ~(size_t)15));  // [M][128] inbox of the cluster reduction
  float *corr = part + M * TILE_N;  // [2 * stages of this slice][MB]

  if (threadIdx.x == 0) {
    for (int i = 0; i < D; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * (D + i)), "r"(T_CWARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 16) reinterpret_cast<uint4 *>(misc)[threadIdx.x] = make_uint4(0, 0, 0, 0);
  if (cs > 1) cluster_arrive_started();
  pdl_launch_dependents();
  __syncthreads();

  if (warp == T_CWARPS) {
    // ---- producer: one thread keeps the ring full -----------------------------------------------------
    if (lane == 0) {
      int slot = 0, round = 0;
      for (int i = 0; i < nst; ++i) {
        if (round > 0 && !t_mbar_wait(bars + 8 * (D + slot), (round - 1) & 1, p.wait_polls)) {
          atomicExch(p.status, 300 + slot);  // site 300: a ring stage was never released
          break;
        }
        const uint32_t full = bars + 8 * slot;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(T_W_BYTES + T_S_BYTES) : "memory");
        const int row = (st_begin + i) * 32;
#pragma unroll
        for (int b = 0; b < 4; ++b) t_tma_2d(ring_w + slot * T_W_BYTES + b * T_BOX_BYTES, &tm_w, tile_n0 + b * 32, row, full);
        t_tma_2d(ring_s + slot * T_S_BYTES, &tm_s, tile_n0, (st_begin + i) * 2, full);
        if (++slot == D) {
          slot = 0;
          ++round;
        }
      }
    }
  } else {
    // ---- consumers ----------------------------------------------------------------------------------------
    const int wn = warp % T_WN, wk = warp / T_WN;
    const int g = lane >> 2, t = lane & 3;
    const int chunk = ((g & 1) << 2) | (g >> 1);  // 16-byte chunk (4 columns) of the warp's 32-column box
    pdl_wait();  // x (and a residual output) may come from the kernel before this one

    // x for this CTA's stages, permuted per packed row to (x0,x4)(x1,x5)(x2,x6)(x3,x7); the words
    // that meet high nibbles (.y, .w) divided by 16; rows at or beyond K are zeros.
    const int rows = nst * 32;
    const int rows_valid = (K - k_begin) / 8 < rows ? (K - k_begin) / 8 : rows;
    auto stage_row = [&](uint4 o, int m, int r, bool inside) {
      const float2 f0 = __half22float2(u2h2(o.x)), f1 = __half22float2(u2h2(o.y)), f2 = __half22float2(u2h2(o.z)), f3 = __half22float2(u2h2(o.w));
      float sx = inside ? ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y)) : 0.f;
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sx += __shfl_xor_sync(0xffffffffu, sx, off);  // 16 packed rows = one group
      {
        uint4 q = make_uint4(0, 0, 0, 0);
        if (inside) {
          q = permute_row(o);
          const __half2 c16th = u2h2(0x2C002C00u);
          q.y = h22u(__hmul2(u2h2(q.y), c16th));
          q.w = h22u(__hmul2(u2h2(q.w), c16th));
        }
        *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = q;
        if (r % 16 == 0) corr[(r / 16) * MB + m] = sx * (-8.0f * 5.9604644775390625e-8f);
      }
    };
    for (int i = threadIdx.x; i < nst * 2 * (MB - M); i += T_CTHREADS)  // batch rows beyond M: zero seed
      corr[(i / (MB - M)) * MB + M + i % (MB - M)] = 0.f;
    const int tid = threadIdx.x;
    if (PRO == PRO_PLAIN) {
      const __half *xg = reinterpret_cast<const __half *>(p.x);
      for (int i = tid; i < M * rows; i += T_CTHREADS) {  // M * rows is a multiple of 32: whole warps
        const int m = i / rows, r = i - m * rows;
        const bool inside = r < rows_valid;
        const uint4 v = inside ? *reinterpret_cast<const uint4 *>(xg + (size_t)m * K + k_begin + r * 8) : make_uint4(0, 0, 0, 0);
        stage_row(v, m, r, inside);
      }
    } else if (PRO == PRO_SILU_MUL) {
      const __half *xg = reinterpret_cast<const __half *>(p.x);
      for (int i = tid; i < M * rows; i += T_CTHREADS) {
        const int m = i / rows, r = i - m * rows;
        const bool inside = r < rows_valid;
        uint32_t o[4] = {0, 0, 0, 0};
        if (inside) {
          const uint4 gv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + k_begin + r * 8);
          const uint4 uv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + K + k_begin + r * 8);
          const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
            o[j] = h22u(__floats2half2_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y));
          }
        }
        stage_row(make_uint4(o[0], o[1], o[2], o[3]), m, r, inside);
      }
    } else {  // RMSNorm of the fp32 row: every CTA recomputes the row's sum of squares (16 KiB from L2 at K = 4096)
      const float *xg = reinterpret_cast<const float *>(p.x);
      const int rowsK = K / 8;
      for (int m = 0; m < M; ++m) {
        float ss = 0.f;
        for (int r = tid; r < rowsK; r += T_CTHREADS) {
          const float4 a = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8);
          const float4 b = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8 + 4);
          ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) sh_ss[warp] = ss;
        asm volatile("bar.sync 1, %0;" ::"n"(T_CTHREADS) : "memory");
        float tot = (lane < T_CWARPS) ? sh_ss[lane] : 0.f;
        tot = warp_sum(tot);
        asm volatile("bar.sync 1, %0;" ::"n"(T_CTHREADS) : "memory");
        const float rs = rsqrtf(tot * (1.0f / (float)K) + p.eps);
        for (int r = tid; r < rows; r += T_CTHREADS) {  // rows is a multiple of 32: whole warps
          const bool inside = r < rows_valid;
          uint4 o = make_uint4(0, 0, 0, 0);
          if (inside) {
            const float *xr = xg + (size_t)m * K + k_begin + r * 8;
            const float4 a = *reinterpret_cast<const float4 *>(xr), b = *reinterpret_cast<const float4 *>(xr + 4);
            const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + k_begin + r * 8);
            const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)),
                         w3 = __half22float2(u2h2(wv.w));
            o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
            o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
            o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
            o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
          }
          stage_row(o, m, r, inside);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(T_CTHREADS) : "memory");

    // per-lane operand addresses
    const unsigned char *xp[NB];
    uint32_t x_adv[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int m = g + nb * 8;
      const bool ok = m < M;
      xp[nb] = ok ? reinterpret_cast<const unsigned char *>(xs) + (size_t)(m * xs_stride) * 2 + wk * 256 + t * 16 : misc + t * 16;
      x_adv[nb] = ok ? 512u : 0u;
    }
    const float *cp = corr + wk * MB + 2 * t;
    // weights: packed row wk*16 + 4s + t of box wn; the swizzle XORs the chunk with (row & 7) = 4(s&1) + t
    const uint32_t w_row = (uint32_t)(wn * T_BOX_BYTES + wk * 2048 + t * 128);
    const uint32_t w_off0 = w_row + (uint32_t)((chunk ^ t) << 4), w_off1 = w_row + (uint32_t)((chunk ^ t ^ 4) << 4);
    const uint32_t s_off = (uint32_t)(wk * 256 + (wn * 32 + chunk * 4) * 2);

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
      if (alive && !t_mbar_wait(bars + 8 * slot, round & 1, p.wait_polls)) {
        if (lane == 0) atomicExch(p.status, 310 + slot);  // site 310: a ring stage never arrived
        alive = false;                                    // stop waiting; the result is void
      }
      const unsigned char *wsrc = ring_wp + slot * T_W_BYTES;
      float d[NB][2][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const float2 seed = *reinterpret_cast<const float2 *>(cp + nb * 8);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          d[nb][j][0] = d[nb][j][2] = seed.x;
          d[nb][j][1] = d[nb][j][3] = seed.y;
        }
      }
      uint4 wv[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) wv[s] = *reinterpret_cast<const uint4 *>(wsrc + s * 512 + ((s & 1) ? w_off1 : w_off0));
      const uint2 sv = *reinterpret_cast<const uint2 *>(ring_sp + slot * T_S_BYTES + s_off);
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        uint4 xc[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) xc[nb] = *reinterpret_cast<const uint4 *>(xp[nb] + s * 64);
        const uint32_t wr[4] = {wv[s].x, wv[s].y, wv[s].z, wv[s].w};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t lo[4], hi[4];
          unpack_pair_raw(wr[2 * j], wr[2 * j + 1], lo, hi);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            mma16816p(d[nb][j], lo[0], lo[1], lo[2], lo[3], xc[nb].x, xc[nb].y);
            mma16816p(d[nb][j], hi[0], hi[1], hi[2], hi[3], xc[nb].z, xc[nb].w);
          }
        }
      }
      // the stage's operands are in registers: hand the slot back
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bars + 8 * (D + slot)) : "memory");
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
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) xp[nb] += x_adv[nb];
      cp += 2 * MB;
      if (++slot == D) {
        slot = 0;
        ++round;
      }
    }

    asm volatile("bar.sync 1, %0;" ::"n"(T_CTHREADS) : "memory");  // every consumer is done with the ring: `red` may overwrite it
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
  for (int i = threadIdx.x; i < M * TILE_N; i += T_THREADS) {
    const int m = i / TILE_N, c = i - m * TILE_N;
    const float v = red[i] + red[M * TILE_N + i];
    const int owner = c / cols_per, cc = c - owner * cols_per;
    float *inbox = (cs > 1) ? cluster.map_shared_rank(part, owner) : part;
    inbox[(krank * M + m) * cols_per + cc] = v;
  }
  if (cs > 1) cluster.sync(); else __syncthreads();
  for (int i = threadIdx.x; i < M * cols_per; i += T_THREADS) {
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

typedef CUresult (*TmaEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

void *tensor_map_encoder();
static TmaEncodeFn tma_encoder() { return reinterpret_cast<TmaEncodeFn>(tensor_map_encoder()); }
// cuTensorMapEncodeTiled, fetched through the runtime (no link against the driver library); nullptr if absent
void *tensor_map_encoder() {
  static TmaEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TmaEncodeFn>(ptr);
    (void)cudaGetLastError();
  }
  return reinterpret_cast<void *>(fn);
}

static unsigned g_tma_wait_polls = 1u << 22;

bool gemv_tma_eligible(int dtype, int M, int K, int N, int group) {
  return dtype == AB200_F16 && group == 128 && K % 128 == 0 && N % 8 == 0 && M >= 1 && M <= 16 && tma_encoder() != nullptr;
}

struct TmaPlan {
  int cs, depth, xs_stride;
  size_t smem;
};

static bool tma_plan(int M, int MB, int stages, int tiles, TmaPlan &pl) {
  const int sms = sm_count();
  int cs = gemv_tuning_cluster();
  if (cs <= 0) {
    // largest K split that keeps every CTA resident at once (3 per SM) and leaves each CTA a stage
    cs = 1;
    while (cs < 8 && tiles * cs * 2 <= 3 * sms && stages / (cs * 2) >= 1) cs *= 2;
  }
  while (cs > 1 && stages / cs < 1) cs /= 2;
  for (;; cs *= 2) {
    const int st_max = (stages + cs - 1) / cs;
    const int xs_stride = st_max * T_STAGE_K + T_XS_PAD;
    const size_t misc = 1024 + 256 + 256 + (((size_t)M * xs_stride * 2 + 15) & ~(size_t)15) + (size_t)M * TILE_N * sizeof(float) +
                        (size_t)2 * st_max * MB * sizeof(float);
    int per_sm = (tiles * cs + sms - 1) / sms;
    if (per_sm > 3) per_sm = 3;
    // prefer every CTA resident at once; with many batch rows the activations crowd the ring out,
    // then fewer CTAs per SM with a deeper ring each
    for (; per_sm >= 1; --per_sm) {
      const size_t budget = (size_t)227 * 1024 / per_sm - 1024;  // 1 KiB per CTA is reserved by the system
      int depth = (budget > misc) ? (int)((budget - misc) / (T_W_BYTES + T_S_BYTES)) : 0;
      if (depth > st_max) depth = st_max;
      if (depth > T_MAX_DEPTH) depth = T_MAX_DEPTH;
      if (depth >= 2 || (depth >= 1 && st_max == 1)) {
        pl.cs = cs;
        pl.depth = depth;
        pl.xs_stride = xs_stride;
        pl.smem = misc + (size_t)depth * (T_W_BYTES + T_S_BYTES);
        return true;
      }
    }
    if (cs >= 8 || stages / (cs * 2) < 1) return false;
  }
}

template <int MB, int PRO, int EPI>
static int launch_tma(const CUtensorMap &tm_w, const CUtensorMap &tm_s, TmaGemvParams p, const TmaPlan &pl, int tiles, cudaStream_t stream) {
  auto kern = w4a16_gemv_tma_kernel<MB, PRO, EPI>;
  if (pl.smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * pl.cs, 1, 1);
  cfg.blockDim = dim3(T_THREADS, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_s, p));
  return AB200_OK;
}

template <int PRO, int EPI>
static int tma_by_batch(const CUtensorMap &tm_w, const CUtensorMap &tm_s, const TmaGemvParams &p, const TmaPlan &pl, int tiles, cudaStream_t s) {
  return (p.M <= 8) ? launch_tma<8, PRO, EPI>(tm_w, tm_s, p, pl, tiles, s) : launch_tma<16, PRO, EPI>(tm_w, tm_s, p, pl, tiles, s);
}

template <int PRO>
static int tma_by_epi(const CUtensorMap &tm_w, const CUtensorMap &tm_s, const TmaGemvParams &p, const TmaPlan &pl, int tiles, int epi,
                      cudaStream_t s) {
  if (epi == EPI_STORE) return tma_by_batch<PRO, EPI_STORE>(tm_w, tm_s, p, pl, tiles, s);
  if (epi == EPI_RESIDUAL) return tma_by_batch<PRO, EPI_RESIDUAL>(tm_w, tm_s, p, pl, tiles, s);
  return tma_by_batch<PRO, EPI_STORE_F32>(tm_w, tm_s, p, pl, tiles, s);
}

// Sets *handled when this variant took the call; otherwise (shape outside the variant, no tensor-map
// encoder in the driver) returns AB200_OK with *handled false and the caller uses another kernel.
int gemv_tma_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                      int K, int N, int group, int epi, cudaStream_t s, bool *handled) {
  *handled = false;
  if (!gemv_tma_eligible(AB200_F16, M, K, N, group)) return AB200_OK;
  const int stages = (K + T_STAGE_K - 1) / T_STAGE_K, tiles = (N + TILE_N - 1) / TILE_N;
  TmaPlan pl;
  if (!tma_plan(M, M <= 8 ? 8 : 16, stages, tiles, pl)) return AB200_OK;
  TmaEncodeFn enc = tma_encoder();
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
  TmaGemvParams p{x, norm_w, out, kernel_error_ptr(), M, K, N, stages, pl.xs_stride, pl.depth, eps, g_tma_wait_polls};
  if (!p.status) return fail(AB200_ECUDA, "w4a16_gemv: status word unavailable");
  *handled = true;
  if (pro == PRO_PLAIN) return tma_by_epi<PRO_PLAIN>(tm_w, tm_s, p, pl, tiles, epi, s);
  if (pro == PRO_RMSNORM) return tma_by_epi<PRO_RMSNORM>(tm_w, tm_s, p, pl, tiles, epi, s);
  return tma_by_epi<PRO_SILU_MUL>(tm_w, tm_s, p, pl, tiles, epi, s);
}

}  // namespace ab200

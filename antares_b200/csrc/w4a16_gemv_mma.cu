// W4A16 decode GEMV, cluster warp-MMA variant (fp16 activations/scales), batch 1..16, K % 128 == 0.
//
// Why warp MMA: on sm_100 the integer/logic pipe and the FP16 pipe both issue at half rate, so a
// GEMV that multiplies on the scalar pipes (w4a16_gemv.cu, ~23 instructions per packed word)
// saturates instruction issue near 45% of HBM bandwidth.  Here every dequantised nibble goes
// through `mma.sync.m16n8k16` (fp16 x fp16 -> fp32) as a raw bit pattern: `w & 0x000F000F` is the
// pair of fp16 subnormals (q * 2^-24), `w & 0x00F000F0` the pair (16q * 2^-24), so the scalar pipes
// only shift and mask (1 SHF + 4 LOP3 per word, nothing on the FP16 pipe), independent of the
// batch size.  The matching x values are stored divided by 16 for the high nibbles, the
// zero-point enters as the accumulator seed -8 * sum(x) * 2^-24 per scale group, and the fp32 sums
// are multiplied by 2^24 once at the end; products are exact in the fp32 accumulators.  The weights are the A operand (16 output columns x 16 k), the activations
// the B operand (16 k x 8 batch rows); batch rows beyond M read a zero block.
//
// Data path: unchanged HBM layout (qweight int32 [K/8, N]).  A warp owns 32 columns; lane
// (g = lane/4, t = lane%4) copies the 16-byte chunk g (4 columns) of packed row 4s+t, so one warp
// instruction reads 4 rows x 128 contiguous bytes.  The stream is `cp.async` (16 B, L2 only) into
// a per-warp shared-memory ring DEPTH blocks (128 k x 32 columns = 2 KiB) deep; each lane reads
// back only what it copied, so completion is tracked with cp.async groups and no barrier.  The
// four lanes of an MMA thread group hold different packed rows: one MMA contracts 16 k-values
// taken from 4 packed rows x the nibble pairs (k0,k4)(k1,k5) [or (k2,k6)(k3,k7)]; x is staged in
// shared memory in that order.  MMA accumulators hold un-scaled sums of one quantisation group
// and are folded into fp32 running sums with the group scale.
//
// The streaming loop is pointer bumping only: no multiplies, no divisions, no bounds predicates
// (out-of-range columns are clamped to the last valid chunk and dropped at the store).
// CTA = 128 columns (4 column warps) x 2 K warps; the K slices of a column tile form a cluster and
// meet in distributed shared memory in fixed order (deterministic; no scratch, no atomics).
// Prologues/epilogues as in the other variants (plain / RMSNorm / SiLU*up; fp16 / residual / fp32).
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int MMA_WN = 4;  // column warps: 4 x 32 columns = TILE_N
constexpr int MMA_WK = 2;  // K warps
constexpr int MMA_WARPS = MMA_WN * MMA_WK;
constexpr int MMA_THREADS = MMA_WARPS * 32;
constexpr int BLK_STEPS = 4;                           // steps (4 packed rows = 32 k) per 128-k block
constexpr int XS_PAD = 32;                             // halves: batch rows 64 B apart modulo 128 B -> conflict-free LDS.128
constexpr int SLOT_BYTES = BLK_STEPS * 512 + 4 * 256;  // weights [4 steps][32 lanes][16 B] + scales [<=4][32 lanes][8 B]

struct MmaGemvParams {
  const void *x;
  const __half *norm_w;
  const int32_t *qw;
  const __half *scales;
  void *out;
  int M, K, N, group;
  int blocks;     // K / 128
  int xs_stride;  // halves between batch rows of x in shared memory; the same in every CTA of a
                  // cluster, so that `part` sits at one offset cluster-wide
  float eps;
};

// MB = 8 (batch <= 8) or 16.  SPG = steps per scale group inside a block: 4 (group % 128 == 0), 2 (64), 1 (32).
template <int MB, int SPG, int PRO, int EPI, int DEPTH>
__global__ void __launch_bounds__(MMA_THREADS) w4a16_gemv_mma_kernel(MmaGemvParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ float sh_ss[MMA_WARPS];
  constexpr int NB = MB / 8;  // B-fragment sets
  constexpr int NSC = BLK_STEPS / SPG;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wn = warp % MMA_WN, wk = warp / MMA_WN;
  const int g = lane >> 2, t = lane & 3;
  const int tile_n0 = tile * TILE_N;
  const int M = p.M, N = p.N, K = p.K;

  // this CTA's K slice in 128-k blocks, and this warp's blocks bb + wk, bb + wk + WK, ...
  const int bb = (int)((long)p.blocks * krank / cs), be = (int)((long)p.blocks * (krank + 1) / cs);
  const int nblk = (be - bb - wk + MMA_WK - 1) / MMA_WK;
  const int k_begin = bb * 128, kslice = (be - bb) * 128;
  const int xs_stride = p.xs_stride;

  // shared memory: [256 B zeros][x rows][red][part][rings]
  __half *xs = reinterpret_cast<__half *>(smem_raw + 256);
  float *red = reinterpret_cast<float *>(smem_raw + 256 + (((size_t)M * xs_stride * 2 + 15) & ~(size_t)15));  // [WK][M][128]
  float *part = red + MMA_WK * M * TILE_N;                                                                    // [M][128]
  float *corr = part + M * TILE_N;  // [fold units of this slice][MB]: -8 * sum(x) * 2^-24 per fold unit and batch row
  const unsigned char *ring_p = reinterpret_cast<const unsigned char *>(corr + (size_t)(p.xs_stride - XS_PAD) / 128 * NSC * MB) + warp * (DEPTH * SLOT_BYTES) + lane * 16;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_p);

  pdl_launch_dependents();
  if (threadIdx.x < 16) reinterpret_cast<uint4 *>(smem_raw)[threadIdx.x] = make_uint4(0, 0, 0, 0);

  // ---- weight stream: bumped pointers ------------------------------------------------------------------
  int n0 = tile_n0 + wn * 32 + g * 4;  // this thread's 4 columns
  const bool col_ok = n0 < N;
  if (!col_ok) n0 = N - 4;             // clamp: loads stay in range, the result is dropped
  const int b_first = bb + wk;
  const uint4 *wp = reinterpret_cast<const uint4 *>(p.qw + (size_t)(b_first * 16 + t) * N + n0);
  const unsigned w_step = (unsigned)N;  // uint4 elements between packed rows r and r + 4
  const unsigned w_skip = (unsigned)N * 4u * (MMA_WK - 1);  // over the blocks of the other K warps
  // scale rows: SPG == 4: one row per `gb` blocks (gb = group / 128); else 128/group rows per block
  const int gb = (SPG == 4) ? p.group / 128 : 1;
  const int rows_per_blk = (SPG == 4) ? 1 : 128 / p.group;
  int sblk = b_first;  // block whose scales `sp` points at
  const __half *sp = p.scales + (size_t)((SPG == 4) ? (b_first / gb) : (b_first * rows_per_blk)) * N + n0;
  auto issue_block = [&](int slot) {
    const uint32_t dst = ring + slot * SLOT_BYTES;
#pragma unroll
    for (int s = 0; s < BLK_STEPS; ++s) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + s * 512), "l"(wp) : "memory");
      wp += w_step;
    }
    wp += w_skip;
    const uint32_t sdst = dst - lane * 8u + BLK_STEPS * 512;
#pragma unroll
    for (int i = 0; i < NSC; ++i)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sdst + i * 256), "l"(sp + (size_t)i * N) : "memory");
    if (SPG == 4) {
      if (gb == 1) {
        sp += (size_t)N * MMA_WK;
      } else {
        const int nxt = sblk + MMA_WK;
        sp += (size_t)N * (nxt / gb - sblk / gb);
        sblk = nxt;
      }
    } else {
      sp += (size_t)N * rows_per_blk * MMA_WK;
    }
  };
#pragma unroll
  for (int i = 0; i < DEPTH; ++i) {  // the first DEPTH blocks are on their way before x exists
    if (i < nblk) issue_block(i);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  pdl_wait();  // x (and a residual output) may come from the kernel before this one

  // ---- prologue: this CTA's slice of x, permuted per packed row to (x0,x4)(x1,x5)(x2,x6)(x3,x7) ---------
  // The nibbles enter the MMA as raw fp16 bit patterns (subnormals q * 2^-24; the high nibble of a
  // byte is 16q * 2^-24), so the x values that meet high nibbles - words .y and .w of a permuted
  // row - are stored divided by 16, and the zero-point becomes -8 * sum(x) per fold unit
  // (SPG * 32 k), which seeds the MMA accumulators.
  const int rows = kslice / 8;
  constexpr int FOLD_ROWS = SPG * 4;  // packed rows per fold unit (4, 8 or 16 lanes of a warp)
  auto stage_row = [&](uint4 o, int m, int r, bool valid) {
    const float2 f0 = __half22float2(u2h2(o.x)), f1 = __half22float2(u2h2(o.y)), f2 = __half22float2(u2h2(o.z)), f3 = __half22float2(u2h2(o.w));
    float sx = valid ? ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y)) : 0.f;
#pragma unroll
    for (int off = FOLD_ROWS / 2; off > 0; off >>= 1) sx += __shfl_xor_sync(0xffffffffu, sx, off);
    if (valid) {
      uint4 q = permute_row(o);
      const __half2 c16th = u2h2(0x2C002C00u);
      q.y = h22u(__hmul2(u2h2(q.y), c16th));
      q.w = h22u(__hmul2(u2h2(q.w), c16th));
      *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = q;
      if (r % FOLD_ROWS == 0) corr[(r / FOLD_ROWS) * MB + m] = sx * (-8.0f * 5.9604644775390625e-8f);
    }
  };
  for (int i = threadIdx.x; i < (be - bb) * NSC * (MB - M); i += MMA_THREADS)  // batch rows beyond M: zero seed
    corr[(i / (MB - M)) * MB + M + i % (MB - M)] = 0.f;
  const int stage_n = (M * rows + 31) & ~31;
  if (PRO == PRO_PLAIN) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < stage_n; i += MMA_THREADS) {
      const bool valid = i < M * rows;
      const int m = valid ? i / rows : 0, r = valid ? i - m * rows : 0;
      stage_row(*reinterpret_cast<const uint4 *>(xg + (size_t)m * K + k_begin + r * 8), m, r, valid);
    }
  } else if (PRO == PRO_SILU_MUL) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < stage_n; i += MMA_THREADS) {
      const bool valid = i < M * rows;
      const int m = valid ? i / rows : 0, r = valid ? i - m * rows : 0;
      const uint4 gv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + k_begin + r * 8);
      const uint4 uv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + K + k_begin + r * 8);
      const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
        o[j] = h22u(__floats2half2_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y));
      }
      stage_row(make_uint4(o[0], o[1], o[2], o[3]), m, r, valid);
    }
  } else {  // RMSNorm of the fp32 row: every CTA recomputes the row's sum of squares (16 KiB from L2 at K = 4096)
    const float *xg = reinterpret_cast<const float *>(p.x);
    const int rowsK = K / 8;
    const int rows_pad = (rows + 31) & ~31;
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int r = threadIdx.x; r < rowsK; r += MMA_THREADS) {
        const float4 a = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8);
        const float4 b = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8 + 4);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) sh_ss[warp] = ss;
      __syncthreads();
      float tot = (lane < MMA_WARPS) ? sh_ss[lane] : 0.f;
      tot = warp_sum(tot);
      __syncthreads();
      const float rs = rsqrtf(tot * (1.0f / (float)K) + p.eps);
      for (int r0 = threadIdx.x; r0 < rows_pad; r0 += MMA_THREADS) {
        const bool valid = r0 < rows;
        const int r = valid ? r0 : 0;
        const float *xr = xg + (size_t)m * K + k_begin + r * 8;
        const float4 a = *reinterpret_cast<const float4 *>(xr), b = *reinterpret_cast<const float4 *>(xr + 4);
        const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + k_begin + r * 8);
        const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)),
                     w3 = __half22float2(u2h2(wv.w));
        uint4 o;
        o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
        o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
        o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
        o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
        stage_row(o, m, r, valid);
      }
    }
  }
  __syncthreads();

  // ---- streaming loop --------------------------------------------------------------------------------------
  // Byte address of this lane's x operand for its first block; lanes whose batch row is beyond M
  // read the zero block and never advance.
  const uint32_t xs_base = (uint32_t)__cvta_generic_to_shared(xs);
  const uint32_t zero_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  uint32_t xa[NB], x_adv[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = g + nb * 8;
    const bool ok = m < M;
    xa[nb] = ok ? xs_base + (uint32_t)(m * xs_stride) * 2u + (uint32_t)(wk * 256) + t * 16u : zero_base + t * 16u;
    x_adv[nb] = ok ? 256u * MMA_WK : 0u;
  }

  float facc[NB][2][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) facc[nb][j][i] = 0.f;

  // x operand pointers (generic pointers into shared memory: plain loads, so the compiler can
  // hoist them over the MMAs of the step before)
  const unsigned char *xp[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) xp[nb] = smem_raw + (xa[nb] - zero_base);

  // accumulator seeds of this lane's batch rows 2t, 2t+1 (per B-fragment set), first block of this warp
  const float *cp = corr + wk * NSC * MB + 2 * t;

  auto compute_block = [&](int slot) {
    const unsigned char *src = ring_p + slot * SLOT_BYTES;
    float d[NB][2][4];
    uint4 wv = *reinterpret_cast<const uint4 *>(src);
    uint4 xb[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) xb[nb] = *reinterpret_cast<const uint4 *>(xp[nb]);
#pragma unroll
    for (int s = 0; s < BLK_STEPS; ++s) {
      if (s % SPG == 0) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const float2 seed = *reinterpret_cast<const float2 *>(cp + (s / SPG) * MB + nb * 8);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            d[nb][j][0] = d[nb][j][2] = seed.x;
            d[nb][j][1] = d[nb][j][3] = seed.y;
          }
        }
      }
      const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
      uint4 xc[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) xc[nb] = xb[nb];
      if (s + 1 < BLK_STEPS) {  // next step's operands are requested before this step's math
        wv = *reinterpret_cast<const uint4 *>(src + (s + 1) * 512);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) xb[nb] = *reinterpret_cast<const uint4 *>(xp[nb] + (s + 1) * 64);
      }
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
      if (s % SPG == SPG - 1) {
        const uint2 sv = *reinterpret_cast<const uint2 *>(src - lane * 8 + BLK_STEPS * 512 + (s / SPG) * 256);
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
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) xp[nb] += x_adv[nb];
    cp += MMA_WK * NSC * MB;
  };

  for (int i0 = 0; i0 < nblk; i0 += DEPTH) {
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) {
      if (i0 + i < nblk) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");  // this thread's copies of block i0+i landed
        compute_block(i);
        if (i0 + i + DEPTH < nblk) issue_block(i);  // refill the slot just drained (same thread wrote and read it)
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- reduction: K warps -> CTA partial -> cluster (fixed order) -> epilogue ------------------
  // facc[nb][j][i]: column wn*32 + g*4 + 2j + (i>>1), batch nb*8 + 2t + (i&1).
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = nb * 8 + 2 * t + (i & 1);
        if (m < M) red[(wk * M + m) * TILE_N + wn * 32 + g * 4 + 2 * j + (i >> 1)] = col_ok ? facc[nb][j][i] * 16777216.0f : 0.f;
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
    if (n < N) {
      if (EPI == EPI_STORE) reinterpret_cast<__half *>(p.out)[(size_t)m * N + n] = __float2half_rn(s);
      else if (EPI == EPI_STORE_F32) reinterpret_cast<float *>(p.out)[(size_t)m * N + n] = s;
      else reinterpret_cast<float *>(p.out)[(size_t)m * N + n] += __half2float(__float2half_rn(s));
    }
  }
  if (cs > 1) cluster.sync();
}

// ---- host side -------------------------------------------------------------------------------

struct GemvTuning {
  int cluster = 0;  // 0 = heuristic
  int impl = 0;     // 0 = auto, 1 = scalar pipes, 2 = cluster warp MMA, 3 = persistent warp MMA
  int depth = 0;    // 0 = default ring depth
};
static GemvTuning g_tune;

static int pick_cluster_mma(int tiles, int blocks) {
  if (g_tune.cluster > 0) return g_tune.cluster;
  const int target = 4 * sm_count();
  int cs = 1;
  while (cs < 8 && tiles * cs < target && blocks / (cs * 2) >= MMA_WK) cs *= 2;
  return cs;
}

template <typename Kern>
static int launch_mma(Kern kern, MmaGemvParams p, int depth, cudaStream_t stream) {
  const size_t ring_bytes = (size_t)MMA_WARPS * depth * SLOT_BYTES;
  const int tiles = (p.N + TILE_N - 1) / TILE_N;
  int cs = pick_cluster_mma(tiles, p.blocks);
  auto smem_for = [&](int c) {
    const int blocks_max = (p.blocks + c - 1) / c;
    return 256 + (((size_t)p.M * (blocks_max * 128 + XS_PAD) * 2 + 15) & ~(size_t)15) + (size_t)(MMA_WK + 1) * p.M * TILE_N * sizeof(float) +
           (size_t)blocks_max * 4 * 16 * sizeof(float) /* seeds: <= 4 fold units per block x 16 batch rows */ + ring_bytes;
  };
  while (smem_for(cs) > 200 * 1024 && cs < 8) cs *= 2;
  const size_t smem = smem_for(cs);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: K=%d x M=%d does not fit shared memory", p.K, p.M);
  p.xs_stride = ((p.blocks + cs - 1) / cs) * 128 + XS_PAD;
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * cs, 1, 1);
  cfg.blockDim = dim3(MMA_THREADS, 1, 1);
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
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return AB200_OK;
}

bool gemv_mma_eligible(int dtype, int M, int K, int N) { return dtype == AB200_F16 && g_tune.impl != 1 && K % 128 == 0 && N >= 4; }

template <int MB, int SPG, int PRO, int EPI>
static int mma_by_depth(const MmaGemvParams &p, cudaStream_t s) {
  switch (g_tune.depth) {
    case 3: return launch_mma(w4a16_gemv_mma_kernel<MB, SPG, PRO, EPI, 3>, p, 3, s);
    case 4: return launch_mma(w4a16_gemv_mma_kernel<MB, SPG, PRO, EPI, 4>, p, 4, s);
    default: return launch_mma(w4a16_gemv_mma_kernel<MB, SPG, PRO, EPI, 2>, p, 2, s);
  }
}

template <int MB, int PRO, int EPI>
static int mma_by_group(const MmaGemvParams &p, cudaStream_t s) {
  if (p.group % 128 == 0) return mma_by_depth<MB, 4, PRO, EPI>(p, s);
  if (p.group % 64 == 0) return launch_mma(w4a16_gemv_mma_kernel<MB, 2, PRO, EPI, 2>, p, 2, s);
  return launch_mma(w4a16_gemv_mma_kernel<MB, 1, PRO, EPI, 2>, p, 2, s);
}

template <int PRO, int EPI>
static int mma_by_batch(const MmaGemvParams &p, cudaStream_t s) {
  return (p.M <= 8) ? mma_by_group<8, PRO, EPI>(p, s) : mma_by_group<16, PRO, EPI>(p, s);
}

template <int PRO>
static int mma_by_epi(const MmaGemvParams &p, int epi, cudaStream_t s) {
  if (epi == EPI_STORE) return mma_by_batch<PRO, EPI_STORE>(p, s);
  if (epi == EPI_RESIDUAL) return mma_by_batch<PRO, EPI_RESIDUAL>(p, s);
  return mma_by_batch<PRO, EPI_STORE_F32>(p, s);
}

int gemv_mma_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                      int K, int N, int group, int epi, cudaStream_t s) {
  MmaGemvParams p{x, norm_w, qw, reinterpret_cast<const __half *>(scales), out, M, K, N, group, K / 128, 0, eps};
  if (pro == PRO_PLAIN) return mma_by_epi<PRO_PLAIN>(p, epi, s);
  if (pro == PRO_RMSNORM) return mma_by_epi<PRO_RMSNORM>(p, epi, s);
  return mma_by_epi<PRO_SILU_MUL>(p, epi, s);
}

int gemv_tuning_set(const char *name, int value) {
  if (!strcmp(name, "gemv_cluster")) {
    if (!(value == 0 || value == 1 || value == 2 || value == 4 || value == 8)) return fail(AB200_EINVAL, "gemv_cluster must be 0, 1, 2, 4 or 8");
    g_tune.cluster = value;
  } else if (!strcmp(name, "comm_wait_polls")) {
    if (value < 1) return fail(AB200_EINVAL, "comm_wait_polls must be positive");
    comm_set_wait_polls((unsigned)value);
  } else if (!strcmp(name, "pdl")) {
    if (value < 0 || value > 2) return fail(AB200_EINVAL, "pdl must be 0 (off), 1 (release dependents at kernel start) or 2 (GEMVs release them after streaming)");
    pdl_set(value);
  } else if (!strcmp(name, "gemv_depth")) {
    if (value != 0 && (value < 2 || value > 4)) return fail(AB200_EINVAL, "gemv_depth must be 0 or 2..4");
    g_tune.depth = value;
  } else if (!strcmp(name, "gemv_impl")) {
    if (value < 0 || value > 7)
      return fail(AB200_EINVAL, "gemv_impl must be 0 (auto), 1 (scalar pipes), 2 (cluster warp MMA), 3 (persistent warp MMA), 4 (TMA ring + warp MMA), 5 (bulk-copy ring, batch 1), 6 (TMA ring with streamed activations, batch 5-16) or 7 (tcgen05 with the weights in tensor memory)");
    g_tune.impl = value;
  } else if (!strcmp(name, "ring_depth")) {
    return gemv_ring_set_depth(value);

  } else {
    return fail(AB200_EINVAL, "unknown option %s", name);
  }
  return AB200_OK;
}

int gemv_tuning_cluster() { return g_tune.cluster; }
int gemv_tuning_impl() { return g_tune.impl; }

}  // namespace ab200

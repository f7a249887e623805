// W4A16 decode GEMV on the 5th-generation tensor cores (fp16, group 128, 1-16 batch rows): weights^T is
// the MMA's A operand, written straight into tensor memory; the activations are the B operand.
// Opt-in (option gemv_impl=7): measured slower than the warp-MMA kernels at these batch sizes, see below.
//
// Replaces the kernel the reference generates from samples/05_llama2_7b_int4.py:135-139.
//
// y^T[n, m] = sum_k W[k, n] x[m, k]: a 128-column tile of the weight matrix gives the 128 rows of a
// `tcgen05.mma.cta_group::1.kind::f16` (M128 N16 K16), the (zero-padded) 16 batch rows give its N.  A packed
// int32 word holds eight consecutive k of one column, which is exactly 16 bytes of one K-major A row, so the
// thread that owns column n (= TMEM lane n) turns each of its words into four registers
//     (w & 0x000F000F, w & 0x00F000F0, (w >> 8) & 0x000F000F, (w >> 8) & 0x00F000F0)
// = the fp16 pairs (q0,q4) (16 q1,16 q5) (q2,q6) (16 q3,16 q7) * 2^-24 (raw nibbles read as subnormals) and
// stores them to tensor memory with `tcgen05.st`: 1 shift + 4 LOP3 per word, and the 4x larger fp16 operand
// never passes through shared memory.  The activations come from a small kernel that writes them once in the
// matching k order, the odd pairs divided by 16, as the K-major core-matrix layout the MMA reads from shared
// memory, one slab per 256-k stage, followed by the accumulator corrections -8 * 2^-24 * sum_k x per
// quantisation group; slabs and scales travel through one TMA ring, the packed weights through another (a
// weight stage is free as soon as its words are in registers, an activation stage only when its MMAs are done).
//
// The tensor core accumulates one quantisation group (128 k = 8 MMAs) in its own 16 TMEM columns; four
// warps read a finished group back (`tcgen05.ld`), add the correction, multiply by the column's scale and
// add into fp32 registers, while the MMAs of the next group run into the other accumulator.
//
// Roles in a CTA of 16 warps: 2 x 4 warps dequantise (group 0 / group 1 of every stage), 4 warps drain
// accumulators, 1 thread runs the TMA rings, 2 threads issue the MMAs (one per group), 1 warp moves finished
// sums to global memory.  They meet only through mbarriers.
//
// Work split: persistent CTAs, two per SM.  The (tile, stage) units in tile-major order are cut into equal
// contiguous ranges, one per CTA; a CTA that finishes its part of a tile stores the partial sums, the last CTA
// to arrive at the tile adds the partials in range order (bitwise repeatable) and writes the output.
// Every wait is bounded (status sites 600-680).
//
// Measured on B200 (gate|up projection 4096 x 22016, isolated, cold weights): 24 us at 1 row, 30 us at 16,
// against 11 us (scalar kernel, 1 row) and 20 us (warp-MMA ring kernel, 16 rows).  Device timestamps put the
// main loop at about 1800 cycles per 256-k stage and CTA (bounded by the two MMA-issuing threads: an M128 N16
// K16 instruction costs its issuing thread about 100 cycles and a stage needs 16 of them), 9 stages per CTA:
// 8.5 us, close to the 7.1 us the bytes take at the measured HBM rate.  The rest is what surrounds the loop: the
// activation kernel in front (launch + run, serialised by the dependency), ring ramp-up behind the TMEM
// allocation, and the exchange of partial sums (3-5 us at 16 rows).  The instruction count does not depend on
// N, so the same structure would pay off at batch sizes well beyond 16.
#include <cuda.h>  // CUtensorMap (types only)

#include "common.cuh"
#include "gemv_shared.cuh"

namespace ab200 {

constexpr int C_DQ_WARPS = 8, C_DRAIN_WARPS = 4;
constexpr int C_PRODUCER_WARP = 12, C_ISSUER_WARP = 13, C_FLUSH_WARP = 15;  // issuers: warps 13 and 14
constexpr int C_THREADS = 16 * 32;
constexpr int C_MB = 16;                          // batch rows of the MMA (N)
constexpr int C_W_BYTES = 32 * TILE_N * 4;        // 32 packed rows x 128 columns
constexpr int C_SC_BYTES = 2 * TILE_N * 2;        // two scale rows
constexpr int C_X_BYTES = 32 * 2 * 128;           // 32 chunks of 8 k x 2 row groups x (8 rows x 16 B)
constexpr int C_SLAB = C_X_BYTES + 2 * C_MB * 4;  // + corrections [2 groups][16]
constexpr int C_XSTAGE = C_SC_BYTES + C_SLAB;     // stage of the activation ring: scales | x | corrections = 8832 = 69 * 128
constexpr int C_DW = 3, C_DX = 5;                 // ring depths: weights (16 KiB stages, held until read into registers),
                                                  // activations (held until the stage's MMAs are complete and drained)
constexpr int C_MAX_DEPTH = 8;
constexpr int C_NA = 3;                           // A buffers (64 k = 32 TMEM columns each) per dequantising warp group
constexpr int C_ND = 2;                           // accumulators (16 TMEM columns each) per group of a stage
constexpr int C_A0_COLS = 128, C_A1_COLS = 64, C_D_COLS = 64;  // TMEM allocations: A buffers 0-3, A buffers 4-5, accumulators
// instruction descriptor: D fp32, A/B fp16, both K-major, N = 16, M = 128
constexpr uint32_t C_IDESC = (1u << 4) | ((uint32_t)(C_MB >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);

struct TcPrepParams {
  const void *x;
  const __half *norm_w;
  unsigned char *slabs;
  int M, K, stages;
  float eps;
};

// One CTA per batch row (rows M..15: zero rows).  Thread = packed rows tid, tid + 256, ...
template <int PRO>
__global__ void __launch_bounds__(256) gemv_tc_prep_kernel(TcPrepParams p) {
  __shared__ float sh[8];
  pdl_launch_dependents();
  pdl_wait();  // the activations come from the kernel before; the slabs may still be read by the GEMV before that one
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int K = p.K, rows_total = p.stages * 32, rows_valid = K / 8;
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
      uint4 q = permute_row(o);  // (x0,x4)(x1,x5)(x2,x6)(x3,x7): the order the nibble masks produce
      const __half2 c16th = u2h2(0x2C002C00u);
      q.y = h22u(__hmul2(u2h2(q.y), c16th));
      q.w = h22u(__hmul2(u2h2(q.w), c16th));
      unsigned char *slab = p.slabs + (size_t)(r / 32) * C_SLAB;
      *reinterpret_cast<uint4 *>(slab + (r % 32) * 256 + (m >> 3) * 128 + (m & 7) * 16) = q;
      if (r % 16 == 0) reinterpret_cast<float *>(slab + C_X_BYTES)[((r % 32) / 16) * C_MB + m] = sx * (-8.0f * 5.9604644775390625e-8f);
    }
  }
}

struct TcGemvParams {
  const unsigned char *slabs;
  void *out;
  int *status;
  float *partial;      // [tiles][max_cnt][M][128]
  unsigned *counters;  // [tiles], zero between launches
  int M, N;
  int S;       // stages per tile = ceil(K / 256)
  int U;       // tiles * S
  int max_cnt; // partial slots per tile
  unsigned wait_polls;
};

__device__ __forceinline__ uint32_t c_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool c_mbar_wait(uint32_t bar, unsigned parity, unsigned polls) {
  {  // non-blocking probe first: the common case is a phase that completed long ago
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
__device__ __forceinline__ void c_mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void c_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// K-major shared-memory operand without swizzle: core matrices of 8 rows x 16 bytes; lbo = bytes between the
// two 16-byte K chunks of one MMA, sbo = bytes between 8-row groups.
__device__ __forceinline__ uint64_t c_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// D[tmem_d] (+)= A[tmem_a] . B[desc]: M128 N16 K16, A from tensor memory
template <bool ACCUMULATE>
__device__ __forceinline__ void c_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t db) {
  if (ACCUMULATE)
    asm volatile("{\n .reg .pred p;\n setp.eq.u32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%4, %4, %4, %4}, p;\n}\n" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(db), "r"(C_IDESC), "r"(0u)
                 : "memory");
  else
    asm volatile("{\n .reg .pred p;\n setp.ne.u32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%4, %4, %4, %4}, p;\n}\n" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(db), "r"(C_IDESC), "r"(0u)
                 : "memory");
}

// The CTAs whose unit ranges meet tile t: first, count
// (U * G fits 32 bits: the host checks it)
__device__ __forceinline__ void c_tile_parts(unsigned U, unsigned G, unsigned S, unsigned t, int &first, int &cnt) {
  const unsigned a = t * S, b = a + S - 1;
  unsigned bf = a * G / U, bl = b * G / U;
  while (bf + 1 < G && U * (bf + 1) / G <= a) ++bf;
  while (bl + 1 < G && U * (bl + 1) / G <= b) ++bl;
  first = (int)bf;
  cnt = (int)(bl - bf) + 1;
}

template <int EPI>
__global__ void __launch_bounds__(C_THREADS, 2) w4a16_gemv_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                                                                      TcGemvParams p) {
  extern __shared__ unsigned char c_smem[];
  // barriers: wfull[8] wempty[8] xfull[8] xempty[8] aready[2][NA] afree[2][NA] dready[2][ND] dfree[2][ND] fready[2] ffree[2]
  __shared__ __align__(8) unsigned long long sh_bars[4 * C_MAX_DEPTH + 4 * C_NA + 4 * C_ND + 4];
  __shared__ uint32_t sh_tmem[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int M = p.M, N = p.N, S = p.S;
  const unsigned U = p.U, G = gridDim.x;
  const int u0 = (int)(U * blockIdx.x / G), u1 = (int)(U * (blockIdx.x + 1) / G);
  const int n_units = u1 - u0;
  const unsigned polls = p.wait_polls;

  // shared memory: [weight ring: DW stages][activation ring: DX stages][flush staging: 2 x [16][128] fp32]
  const uint32_t base_u32 = c_smem_u32(c_smem);
  const uint32_t ring = (base_u32 + 127u) & ~127u;
  unsigned char *ring_p = c_smem + (ring - base_u32);
  const uint32_t xring = ring + C_DW * C_W_BYTES;
  unsigned char *xring_p = ring_p + C_DW * C_W_BYTES;
  float *staging = reinterpret_cast<float *>(xring_p + C_DX * C_XSTAGE);
  const uint32_t bars = c_smem_u32(sh_bars);
  const uint32_t b_wfull = bars, b_wempty = bars + 8 * C_MAX_DEPTH, b_xfull = bars + 16 * C_MAX_DEPTH, b_xempty = bars + 24 * C_MAX_DEPTH,
                 b_aready = bars + 32 * C_MAX_DEPTH, b_afree = b_aready + 16 * C_NA,
                 b_dready = b_afree + 16 * C_NA, b_dfree = b_dready + 16 * C_ND, b_fready = b_dfree + 16 * C_ND, b_ffree = b_fready + 16;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C_MAX_DEPTH; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b_wfull + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(b_wempty + 8 * i), "n"(C_DQ_WARPS));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b_xfull + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(b_xempty + 8 * i), "n"(C_DRAIN_WARPS));
    }
    for (int i = 0; i < 2 * C_NA; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(b_aready + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b_afree + 8 * i));
    }
    for (int i = 0; i < 2 * C_ND; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b_dready + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(b_dfree + 8 * i));
    }
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(b_fready + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b_ffree + 8 * i));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == C_ISSUER_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c_smem_u32(&sh_tmem[0])), "n"(C_A0_COLS) : "memory");
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c_smem_u32(&sh_tmem[1])), "n"(C_A1_COLS) : "memory");
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c_smem_u32(&sh_tmem[2])), "n"(C_D_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_a0 = sh_tmem[0], tmem_a1 = sh_tmem[1], tmem_d = sh_tmem[2];
  // A buffer b of warp group h: index h * NA + b; the first four live in the first allocation
  auto a_addr = [&](int idx) { return idx < 4 ? tmem_a0 + idx * 32 : tmem_a1 + (idx - 4) * 32; };

  if (warp == C_PRODUCER_WARP) {
    // ---- TMA ring --------------------------------------------------------------------------------------------
    int t = u0 / S, s = u0 - t * S;  // tile and stage of the next unit to issue
    auto issue_weights = [&](int slot) {
      const uint32_t full = b_wfull + 8 * slot;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "n"(C_W_BYTES) : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(ring + slot * C_W_BYTES),
                   "l"(reinterpret_cast<uint64_t>(&tm_w)), "r"(t * TILE_N), "r"(s * 32), "r"(full)
                   : "memory");
    };
    auto issue_scales = [&](int slot) {
      const uint32_t full = b_xfull + 8 * slot;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "n"(C_XSTAGE) : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(xring + slot * C_XSTAGE),
                   "l"(reinterpret_cast<uint64_t>(&tm_s)), "r"(t * TILE_N), "r"(s * 2), "r"(full)
                   : "memory");
    };
    auto issue_slab = [&](int slot, int stage) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(xring + slot * C_XSTAGE + C_SC_BYTES),
                   "l"(p.slabs + (size_t)stage * C_SLAB), "n"(C_SLAB), "r"(b_xfull + 8 * slot)
                   : "memory");
    };
    auto next_unit = [&]() {
      if (++s == S) {
        s = 0;
        ++t;
      }
    };
    // first ring fills: weights and scales at once (they never depend on the kernel before), slabs after the wait
    const int t_first = t, s_first = s;
    const int wfirst = n_units < C_DW ? n_units : C_DW, xfirst = n_units < C_DX ? n_units : C_DX;
    if (lane == 0) {
      for (int i = 0; i < xfirst; ++i) {
        if (i < wfirst) issue_weights(i);
        issue_scales(i);
        next_unit();
      }
    }
    pdl_wait();
    if (lane == 0) {
      for (int i = 0, ss = s_first; i < xfirst; ++i) {
        issue_slab(i, ss);
        if (++ss == S) ss = 0;
      }
      // from here on the weight ring runs C_DX - C_DW units behind the activation ring
      int wt = t_first, ws = s_first;  // unit of the next weight stage
      for (int i = 0; i < wfirst; ++i)
        if (++ws == S) {
          ws = 0;
          ++wt;
        }
      int wslot = 0, wph = 0, xslot = 0, xph = 0;
      for (int iw = wfirst, ix = xfirst; iw < n_units; ++iw) {
        if (!c_mbar_wait(b_wempty + 8 * wslot, wph, polls)) {
          atomicExch(p.status, 600 + wslot);  // site 600: a weight stage was never released
          break;
        }
        {
          const int tt = t, sv = s;
          t = wt;
          s = ws;
          issue_weights(wslot);
          t = tt;
          s = sv;
        }
        if (++ws == S) {
          ws = 0;
          ++wt;
        }
        if (++wslot == C_DW) {
          wslot = 0;
          wph ^= 1;
        }
        if (ix < n_units) {
          if (!c_mbar_wait(b_xempty + 8 * xslot, xph, polls)) {
            atomicExch(p.status, 605 + xslot);  // site 605: an activation stage was never released
            break;
          }
          issue_scales(xslot);
          issue_slab(xslot, s);
          next_unit();
          ++ix;
          if (++xslot == C_DX) {
            xslot = 0;
            xph ^= 1;
          }
        }
      }
    }
  } else if (warp == C_ISSUER_WARP || warp == C_ISSUER_WARP + 1) {
    // ---- MMA issue: one thread per quantisation group of a stage -------------------------------------------------
    pdl_wait();
    if (lane == 0) {
      const int h = warp - C_ISSUER_WARP;
      int slot = 0, fph = 0, ab = 0, aph = 0, di = 0, dph = 0;
      for (int i = 0; i < n_units; ++i) {
        if (!c_mbar_wait(b_xfull + 8 * slot, fph, polls)) {
          atomicExch(p.status, 610 + slot);  // site 610: an activation stage never arrived
          break;
        }
        if (i >= C_ND && !c_mbar_wait(b_dfree + 8 * (h * C_ND + di), dph ^ 1, polls)) {
          atomicExch(p.status, 620 + h);  // site 620: an accumulator was never read back
          break;
        }
        const uint64_t db0 = c_desc(xring + slot * C_XSTAGE + C_SC_BYTES + h * 8 * 512, 256, 128);
        const uint32_t td = tmem_d + (h * C_ND + di) * 16;
        bool ok = true;
#pragma unroll
        for (int kbl = 0; kbl < 2; ++kbl) {
          if (!c_mbar_wait(b_aready + 8 * (h * C_NA + ab), aph, polls)) {
            atomicExch(p.status, 630 + h * 2 + kbl);  // site 630: an A block was never written
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t ta = a_addr(h * C_NA + ab);
          const uint64_t db = db0 + (uint64_t)(kbl * 4 * 32);
          if (kbl == 0) c_mma<false>(td, ta, db);
          else c_mma<true>(td, ta, db);
          c_mma<true>(td, ta + 8, db + 32);
          c_mma<true>(td, ta + 16, db + 64);
          c_mma<true>(td, ta + 24, db + 96);
          c_commit(b_afree + 8 * (h * C_NA + ab));
          if (++ab == C_NA) {
            ab = 0;
            aph ^= 1;
          }
        }
        if (!ok) break;
        c_commit(b_dready + 8 * (h * C_ND + di));
        if (++di == C_ND) {
          di = 0;
          dph ^= 1;
        }
        if (++slot == C_DX) {
          slot = 0;
          fph ^= 1;
        }
      }
    }
  } else if (warp < C_DQ_WARPS) {
    // ---- dequantise: packed words -> fp16 A operand in tensor memory --------------------------------------------
    pdl_wait();
    const int h = warp >> 2, q = warp & 3;
    const int n = q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    int slot = 0, fph = 0, ab = 0, aph = 0;
    bool ok = true;
    for (int i = 0; i < n_units && ok; ++i) {
      if (!c_mbar_wait(b_wfull + 8 * slot, fph, polls)) {
        if (lane == 0) atomicExch(p.status, 640 + slot);  // site 640: a weight stage never arrived
        break;
      }
      const uint32_t *wsm = reinterpret_cast<const uint32_t *>(ring_p + (size_t)slot * C_W_BYTES) + (h * 16) * TILE_N + n;
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = wsm[j * TILE_N];
      __syncwarp();
      if (lane == 0) c_mbar_arrive(b_wempty + 8 * slot);  // this warp's words are in registers
#pragma unroll
      for (int kbl = 0; kbl < 2; ++kbl) {
        if (2 * i + kbl >= C_NA && !c_mbar_wait(b_afree + 8 * (h * C_NA + ab), aph ^ 1, polls)) {
          if (lane == 0) atomicExch(p.status, 650 + h * 2 + kbl);  // site 650: the MMAs that read an A block never finished
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ta = a_addr(h * C_NA + ab) + lane_base;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t v = w[kbl * 8 + c * 4 + j], v8 = v >> 8;
            r[4 * j + 0] = v & 0x000F000Fu;
            r[4 * j + 1] = v & 0x00F000F0u;
            r[4 * j + 2] = v8 & 0x000F000Fu;
            r[4 * j + 3] = v8 & 0x00F000F0u;
          }
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(ta + c * 16),
              "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
              "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
              : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) c_mbar_arrive(b_aready + 8 * (h * C_NA + ab));
        if (++ab == C_NA) {
          ab = 0;
          aph ^= 1;
        }
      }
      if (++slot == C_DW) {
        slot = 0;
        fph ^= 1;
      }
    }
  } else if (warp < C_DQ_WARPS + C_DRAIN_WARPS) {
    // ---- drain: accumulators -> scaled fp32 sums -> staging for the flush warp ----------------------------------
    const int q = warp & 3;
    const int n = q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float acc[C_MB];
#pragma unroll
    for (int m = 0; m < C_MB; ++m) acc[m] = 0.f;
    bool ok = true;
    int slot = 0, fph = 0, di = 0, dph = 0, fb = 0, fphase = 0, flushes = 0;
    int s = u0 % S;
    for (int i = 0; i < n_units; ++i) {
      const unsigned char *st = xring_p + (size_t)slot * C_XSTAGE;
      if (ok && !c_mbar_wait(b_xfull + 8 * slot, fph, polls)) ok = false;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (ok && !c_mbar_wait(b_dready + 8 * (h * C_ND + di), dph, polls)) {
          if (lane == 0) atomicExch(p.status, 660 + h);  // site 660: a group's MMAs never finished; the result is void
          ok = false;
        }
        if (!ok) continue;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t d[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]),
              "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
            : "r"(tmem_d + lane_base + (h * C_ND + di) * 16));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) c_mbar_arrive(b_dfree + 8 * (h * C_ND + di));
        const float sc = __half2float(reinterpret_cast<const __half *>(st)[h * TILE_N + n]);
        const float4 *corr = reinterpret_cast<const float4 *>(st + C_SC_BYTES + C_X_BYTES + h * C_MB * 4);
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4) {
          const float4 c = corr[m4];
          acc[4 * m4 + 0] = fmaf(sc, __uint_as_float(d[4 * m4 + 0]) + c.x, acc[4 * m4 + 0]);
          acc[4 * m4 + 1] = fmaf(sc, __uint_as_float(d[4 * m4 + 1]) + c.y, acc[4 * m4 + 1]);
          acc[4 * m4 + 2] = fmaf(sc, __uint_as_float(d[4 * m4 + 2]) + c.z, acc[4 * m4 + 2]);
          acc[4 * m4 + 3] = fmaf(sc, __uint_as_float(d[4 * m4 + 3]) + c.w, acc[4 * m4 + 3]);
        }
      }
      __syncwarp();
      if (lane == 0) c_mbar_arrive(b_xempty + 8 * slot);  // scales and corrections read, the stage's MMAs complete
      if (++di == C_ND) {
        di = 0;
        dph ^= 1;
      }
      if (++slot == C_DX) {
        slot = 0;
        fph ^= 1;
      }
      if (++s == S || i == n_units - 1) {
        // this CTA's part of a tile is complete: hand the sums to the flush warp
        s = 0;
        if (flushes >= 2 && ok && !c_mbar_wait(b_ffree + 8 * fb, fphase ^ 1, polls)) {
          if (lane == 0) atomicExch(p.status, 670 + fb);  // site 670: the flush warp never released a staging buffer
          ok = false;
        }
        float *sg = staging + fb * (C_MB * TILE_N) + n;
#pragma unroll
        for (int m = 0; m < C_MB; ++m) {
          sg[m * TILE_N] = acc[m] * 16777216.0f;
          acc[m] = 0.f;
        }
        __syncwarp();
        if (lane == 0) c_mbar_arrive(b_fready + 8 * fb);
        ++flushes;
        if (++fb == 2) {
          fb = 0;
          fphase ^= 1;
        }
      }
    }
  } else if (warp == C_FLUSH_WARP) {
    // ---- flush: partial sums to global memory; the last CTA to arrive at a tile adds them up and writes the output
    pdl_wait();
    int fb = 0, fphase = 0;
    int t = u0 / S;
    const int t_last = (u1 - 1) / S;
    for (; n_units > 0 && t <= t_last; ++t) {
      if (!c_mbar_wait(b_fready + 8 * fb, fphase, polls)) {
        if (lane == 0) atomicExch(p.status, 680 + fb);  // site 680: sums never arrived
        break;
      }
      int first, cnt;
      c_tile_parts(U, G, (unsigned)S, (unsigned)t, first, cnt);
      const int mine = (int)blockIdx.x - first;
      const float4 *sg = reinterpret_cast<const float4 *>(staging + fb * (C_MB * TILE_N)) + lane;
      const int col = t * TILE_N + lane * 4;
      const bool col_ok = col < N;  // N is a multiple of 8: a lane's four columns are inside or outside together
      auto output = [&](int m, float4 v) {
        if (EPI == EPI_STORE) {
          uint2 o;
          o.x = h22u(__floats2half2_rn(v.x, v.y));
          o.y = h22u(__floats2half2_rn(v.z, v.w));
          *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.out) + (size_t)m * N + col) = o;
        } else if (EPI == EPI_STORE_F32) {
          *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + (size_t)m * N + col) = v;
        } else {
          float4 *o = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + (size_t)m * N + col);
          float4 r = *o;
          r.x += __half2float(__float2half_rn(v.x));
          r.y += __half2float(__float2half_rn(v.y));
          r.z += __half2float(__float2half_rn(v.z));
          r.w += __half2float(__float2half_rn(v.w));
          *o = r;
        }
      };
      if (cnt == 1) {
        for (int m = 0; m < M; ++m) {
          const float4 v = sg[m * (TILE_N / 4)];
          if (col_ok) output(m, v);
        }
      } else {
        float4 *part = reinterpret_cast<float4 *>(p.partial + ((size_t)t * p.max_cnt + mine) * M * TILE_N) + lane;
#pragma unroll
        for (int m0 = 0; m0 < C_MB; m0 += 8) {
          float4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = sg[(m0 + j) * (TILE_N / 4)];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (m0 + j < M) __stcg(part + (m0 + j) * (TILE_N / 4), v[j]);
        }
      }
      __syncwarp();
      if (lane == 0) c_mbar_arrive(b_ffree + 8 * fb);
      if (++fb == 2) {
        fb = 0;
        fphase ^= 1;
      }
      if (cnt > 1) {
        __threadfence();
        __syncwarp();
        unsigned old = 0;
        if (lane == 0) {
          old = atomicAdd(p.counters + t, 1u);
          if (old == (unsigned)(cnt - 1)) p.counters[t] = 0;  // every part of the tile has arrived: ready for the next launch
        }
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == (unsigned)(cnt - 1)) {
          __threadfence();
          const float4 *all = reinterpret_cast<const float4 *>(p.partial + (size_t)t * p.max_cnt * M * TILE_N) + lane;
          for (int m0 = 0; m0 < M; m0 += 4) {  // four rows at a time: their loads are in flight together
            float4 sum[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = 0; c < cnt; ++c) {
              float4 a[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) a[j] = m0 + j < M ? __ldcg(all + ((size_t)c * M + m0 + j) * (TILE_N / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                sum[j].x += a[j].x;
                sum[j].y += a[j].y;
                sum[j].z += a[j].z;
                sum[j].w += a[j].w;
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (col_ok && m0 + j < M) output(m0 + j, sum[j]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == C_ISSUER_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_a0), "n"(C_A0_COLS) : "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_a1), "n"(C_A1_COLS) : "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(C_D_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------

typedef CUresult (*TcEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Library-owned scratch: [counters, zero between launches][slabs][partials]
static int tc_scratch(size_t bytes, void **out) {
  const size_t want = bytes < ((size_t)8 << 20) ? ((size_t)8 << 20) : bytes;
  return library_buffer(LIB_BUF_TC, bytes, want, want, out);
}

constexpr size_t TC_COUNTER_BYTES = 16 * 1024;  // up to 4096 column tiles

bool gemv_tc_eligible(int dtype, int M, int K, int N, int group) {
  return dtype == AB200_F16 && group == 128 && K % 128 == 0 && N % 8 == 0 && M >= 1 && M <= C_MB && (N + TILE_N - 1) / TILE_N <= 4096 &&
         tensor_map_encoder() != nullptr;
}

template <int EPI>
static int launch_tc(const CUtensorMap &tm_w, const CUtensorMap &tm_s, const TcGemvParams &p, int grid, size_t smem, cudaStream_t stream) {
  auto kern = w4a16_gemv_tc_kernel<EPI>;
  AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(C_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_s, p));
  return AB200_OK;
}

// Sets *handled when this variant took the call.
int gemv_tc_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M, int K,
                     int N, int group, int epi, cudaStream_t s, bool *handled) {
  *handled = false;
  if (!gemv_tc_eligible(AB200_F16, M, K, N, group)) return AB200_OK;
  const int S = (K + 255) / 256, tiles = (N + TILE_N - 1) / TILE_N;
  const long U = (long)tiles * S;
  const int sms = sm_count();
  // two CTAs per SM, at least two units per CTA
  long G = 2L * sms;
  if (G > U / 2) G = U / 2;
  if (G < 1) G = 1;
  if (U * (G + 1) >= (1L << 31)) return AB200_OK;  // the kernel's range arithmetic is 32-bit
  const long upc = U / G;  // smallest range
  const int max_cnt = (int)((S + upc - 2) / upc) + 1;
  const size_t smem = 128 + (size_t)C_DW * C_W_BYTES + (size_t)C_DX * C_XSTAGE + 2 * C_MB * TILE_N * sizeof(float);

  const size_t slab_bytes = ((size_t)S * C_SLAB + 255) & ~(size_t)255;
  const size_t part_bytes = (size_t)tiles * max_cnt * M * TILE_N * sizeof(float);
  void *scratch = nullptr;
  if (int rc = tc_scratch(TC_COUNTER_BYTES + slab_bytes + part_bytes, &scratch)) return rc;
  unsigned char *sb = reinterpret_cast<unsigned char *>(scratch);

  TcEncodeFn enc = reinterpret_cast<TcEncodeFn>(tensor_map_encoder());
  CUtensorMap tm_w, tm_s;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 8)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    const cuuint32_t box[2] = {TILE_N, 32}, estr[2] = {1, 1};
    const CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(qw), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
  TcPrepParams pp{x, norm_w, sb + TC_COUNTER_BYTES, M, K, S, eps};
  cudaError_t e;
  if (pro == PRO_PLAIN) e = launch_pdl(gemv_tc_prep_kernel<PRO_PLAIN>, dim3(C_MB), dim3(256), 0, s, pp);
  else if (pro == PRO_RMSNORM) e = launch_pdl(gemv_tc_prep_kernel<PRO_RMSNORM>, dim3(C_MB), dim3(256), 0, s, pp);
  else e = launch_pdl(gemv_tc_prep_kernel<PRO_SILU_MUL>, dim3(C_MB), dim3(256), 0, s, pp);
  if (e != cudaSuccess) return fail(AB200_ECUDA, "w4a16_gemv (tensor-memory kernel): %s", cudaGetErrorString(e));
  TcGemvParams p{sb + TC_COUNTER_BYTES, out, status, reinterpret_cast<float *>(sb + TC_COUNTER_BYTES + slab_bytes),
                 reinterpret_cast<unsigned *>(sb), M, N, S, (int)U, max_cnt, 1u << 22};
  if (epi == EPI_STORE) return launch_tc<EPI_STORE>(tm_w, tm_s, p, (int)G, smem, s);
  if (epi == EPI_RESIDUAL) return launch_tc<EPI_RESIDUAL>(tm_w, tm_s, p, (int)G, smem, s);
  return launch_tc<EPI_STORE_F32>(tm_w, tm_s, p, (int)G, smem, s);
}

}  // namespace ab200

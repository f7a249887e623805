// W4A16 decode GEMV for sm_100a: out[M,N] = x[M,K] . dequant(qweight[K/8,N], scales[K/group,N]).
// Register-prefetch scalar-pipe kernel (no tensor cores): the default for one batch row (and for up to
// four rows on the tile-major layout), plus the fp32 variant and the host-side choice among the GEMV
// kernels (batch 2-16: TMA ring + warp MMA, w4a16_gemv_tma.cu; bulk-copy ring, w4a16_gemv_ring.cu, on
// request and for the tensor-parallel fused exchange).
//
// Replaces the kernel the reference generates from samples/05_llama2_7b_int4.py:135-139.
//
// Data layout in HBM: the reference's, qweight int32 [K/8, N], N contiguous (one 16-byte load = 4 columns
// x 8 k-values; a warp reads 512 contiguous bytes of one packed row), scales fp16/fp32 [K/group, N]; or
// tile-major [N/128][K/8][128] (ab200_w4a16_gemv_tiled), where what one CTA streams is one contiguous range.
//
// Decomposition: CTA = 128 columns x a contiguous slice of K; its 8 warps take 32-k "units" (4 packed
// rows) round-robin, with two units' loads (8 x 16 B per thread) in flight in registers, the first ones
// issued before griddepcontrol.wait and before x is staged.  The K slices of one column tile are the CTAs
// of one thread-block cluster; every CTA pushes its column sums into the owner CTA's inbox through
// distributed shared memory (split cluster barrier: arrive at kernel start, wait before the first remote
// store), one cluster barrier, rank-ordered sum (deterministic, no global scratch, no atomics).
// HBM-bound by design: algorithmic bytes = K*N/2 + (K/group)*N*2 + M*K*2 + M*N*2.
//
// fp16 arithmetic (raw-nibble multiply): `w & 0x000F000F` is a pair of fp16 subnormals q * 2^-24
// (`w & 0x00F000F0` = 16 q * 2^-24); they are multiplied on the FP16 pipe by activations pre-scaled by a
// power of two chosen per batch row (the words that meet high nibbles by another 1/16), 16 products per
// half2 lane, then widened to fp32; the zero-point leaves the inner loop as 8 * sum(x) per 32-k unit,
// subtracted in fp32 before the group scale is applied; everything across units, warps and CTAs is fp32.
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

struct GemvParams {
  const void *x;
  const int32_t *qw;
  const void *scales;
  void *out;
  int K, N, group;
  int units;      // K / 32
  int xs_stride;  // elements between batch rows of x in shared memory (same in every CTA of a cluster)
  const __half *norm_w = nullptr;  // PRO_RMSNORM: fp16 [K]
  float eps = 0.f;
  // L2 prefetch hint: up to two byte ranges (the next projection's packed weights and scales)
  const unsigned char *pf[2] = {nullptr, nullptr};
  unsigned pf_bytes[2] = {0, 0};
  int pdl_late = 0;  // release the dependent kernel after the streaming loop instead of at the start
  // Weight addressing (int32 words / halves): row stride and offset of a 128-column tile.  The
  // reference layout [K/8, N] has ld = N, tile = 128; the tile-major layout [N/128][K/8][128]
  // (each CTA's weights contiguous in HBM) has ld = 128, tile = (K/8) * 128.  0 = reference layout.
  unsigned ld_w = 0, ld_s = 0;
  size_t tile_w = 0, tile_s = 0;
};

constexpr unsigned PF_CHUNK = 16 * 1024;
// One thread per CTA asks the TMA unit to pull this CTA's share of the hinted ranges into L2.
__device__ __forceinline__ void issue_prefetch_hint(const GemvParams &p) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const unsigned bytes = p.pf_bytes[r];
    for (unsigned off = blockIdx.x * PF_CHUNK; off < bytes; off += gridDim.x * PF_CHUNK) {
      const unsigned n = (bytes - off < PF_CHUNK) ? ((bytes - off) & ~15u) : PF_CHUNK;
      if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf[r] + off), "r"(n) : "memory");
    }
  }
}

// PRO selects how x is built in shared memory: plain fp16 x; RMSNorm of an fp32 row (every CTA
// recomputes the row's sum of squares from L2: 16 KiB for K = 4096); SiLU(gate) * up of an fp16
// [M, 2K] row.
template <int M, int EPI, int PRO>
__global__ void __launch_bounds__(GEMV_THREADS) w4a16_gemv_f16_kernel(GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = tile * TILE_N + lane * 4;
  const bool col_ok = n0 < p.N;

  const int u_begin = (int)((long)p.units * krank / cs), u_end = (int)((long)p.units * (krank + 1) / cs);
  const int k_begin = u_begin * UNIT_K, kslice = (u_end - u_begin) * UNIT_K;
  const int xs_stride = p.xs_stride;

  __half *xs = reinterpret_cast<__half *>(smem_raw);
  float *red = reinterpret_cast<float *>(smem_raw + (((size_t)M * xs_stride * 2 + 15) & ~(size_t)15));
  float *part = red + GEMV_WARPS * M * TILE_N;

  // Streaming state: bumped pointers only (no multiplies or divisions per unit, no column
  // predicate: out-of-range columns are clamped to the last valid chunk and dropped at the store).
  const int n0c = col_ok ? n0 : p.N - 4;
  int u = u_begin + warp;
  const unsigned ld_w = p.ld_w ? p.ld_w : (unsigned)p.N, ld_s = p.ld_s ? p.ld_s : (unsigned)p.N;
  const size_t tile_w = p.ld_w ? p.tile_w : (size_t)TILE_N, tile_s = p.ld_s ? p.tile_s : (size_t)TILE_N;
  const int cl = n0c - tile * TILE_N;                                // column offset inside the tile
  const unsigned row_step = ld_w / 4;                                // uint4 elements between packed rows
  const uint4 *wp = reinterpret_cast<const uint4 *>(p.qw + (size_t)tile * tile_w + (size_t)u * UNIT_ROWS * ld_w + cl);
  const unsigned unit_step = row_step * UNIT_ROWS * GEMV_WARPS;     // to this warp's next unit
  // scales: the warp advances 8 units = 256 k per round; for the usual group sizes that is a whole
  // number of scale rows, otherwise the row is recomputed per unit
  const bool s_fast = (UNIT_K * GEMV_WARPS) % p.group == 0;
  const unsigned s_step = (unsigned)((UNIT_K * GEMV_WARPS) / p.group) * ld_s;
  const __half *scol = reinterpret_cast<const __half *>(p.scales) + (size_t)tile * tile_s + cl;
  const __half *sp = scol + (size_t)((u * UNIT_K) / p.group) * ld_s;

  constexpr int NBUF = 2;  // units in flight per warp (registers)
  uint4 wbuf[NBUF][UNIT_ROWS];
  uint2 sbuf[NBUF];
  int u_load = u;  // unit that the next load_unit() fetches
  auto load_unit = [&](int b) {
#pragma unroll
    for (int r = 0; r < UNIT_ROWS; ++r) wbuf[b][r] = ldg_stream_v4(wp + r * row_step);
    sbuf[b] = ldg_nc_v2(sp);
    wp += unit_step;
    u_load += GEMV_WARPS;
    if (s_fast) sp += s_step;
    else sp = scol + (size_t)((u_load * UNIT_K) / p.group) * ld_s;
  };

  if (cs > 1) cluster_arrive_started();
  if (!p.pdl_late) pdl_launch_dependents();
  // the first NBUF units of this warp are on their way before x is staged
#pragma unroll
  for (int b = 0; b < NBUF; ++b)
    if (u_load < u_end) load_unit(b);
  if (threadIdx.x == GEMV_THREADS - 1) issue_prefetch_hint(p);

  // Fast RMSNorm prologue (one batch row, slice of at most 256 packed rows): everything that only
  // needs the constant norm weights happens before the wait - this thread's slice of them, and the
  // largest |w| of the whole row, which bounds the normalised activations.
  const int rows = kslice / 8;
  const bool fast_rms = (M == 1) && (PRO == PRO_RMSNORM) && rows <= GEMV_THREADS;
  __shared__ unsigned sh_wmax[GEMV_WARPS];
  uint4 nw_slice = make_uint4(0, 0, 0, 0);
  if (fast_rms) {
    if ((int)threadIdx.x < rows) nw_slice = __ldg(reinterpret_cast<const uint4 *>(p.norm_w + k_begin) + threadIdx.x);
    unsigned wm = 0u;
    for (int r = threadIdx.x; r < p.K / 8; r += GEMV_THREADS) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.norm_w) + r);
      const unsigned a = v.x & 0x7FFF7FFFu, b = v.y & 0x7FFF7FFFu, c = v.z & 0x7FFF7FFFu, d = v.w & 0x7FFF7FFFu;
      wm = max(wm, max(max(max(a & 0xFFFFu, a >> 16), max(b & 0xFFFFu, b >> 16)), max(max(c & 0xFFFFu, c >> 16), max(d & 0xFFFFu, d >> 16))));
    }
    wm = __reduce_max_sync(0xffffffffu, wm);
    if (lane == 0) sh_wmax[warp] = wm;
  }
  pdl_wait();                      // x (and the output buffer) may come from the kernel before this one

  // Stage this CTA's slice of x into shared memory, permuted so that packed row r holds
  // (x0,x4)(x1,x5)(x2,x6)(x3,x7): the pairing the nibble masks produce.
  //
  // The nibbles meet x as raw fp16 bit patterns: `w & 0x000F000F` is the pair of subnormals
  // (q * 2^-24), `w & 0x00F000F0` the pair (16q * 2^-24).  So that the products stay in fp16's
  // normal range, each batch row of the slice is scaled by a power of two 2^e chosen from its
  // largest magnitude (|x| * 2^e < 2^15); the words that meet high nibbles carry another 1/16.
  // The zero-point becomes 8 * sum(x * 2^e) * 2^-24 per unit, subtracted in fp32, and the fp32
  // row sums are multiplied by 2^(24 - e) before the cross-warp reduction.  Exact powers of two
  // throughout: the only roundings are those of the fp16 product chain, as before.
  auto permute = [](uint4 v) {
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    return o;
  };
  __shared__ unsigned sh_max[M][GEMV_WARPS];
  __shared__ float sh_back[M];  // 2^(24 - e) per batch row
  float *corr = part + M * TILE_N;  // [M][units of the slice]: 8 * 2^-24 * sum over the unit of x * 2^e
  const int n_units = u_end - u_begin;
  if (fast_rms) {
    __shared__ float sh_ss1[GEMV_WARPS], sh_xm1[GEMV_WARPS];
    const float *xg = reinterpret_cast<const float *>(p.x);
    const bool valid = (int)threadIdx.x < rows;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (valid) {
      a = *reinterpret_cast<const float4 *>(xg + k_begin + threadIdx.x * 8);
      b = *reinterpret_cast<const float4 *>(xg + k_begin + threadIdx.x * 8 + 4);
    }
    float ss = 0.f, xm = 0.f;
    for (int r = threadIdx.x; r < p.K / 8; r += GEMV_THREADS) {
      const float4 c = *reinterpret_cast<const float4 *>(xg + r * 8), d = *reinterpret_cast<const float4 *>(xg + r * 8 + 4);
      ss += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w + d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w;
      xm = fmaxf(fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))),
                 fmaxf(xm, fmaxf(fmaxf(fabsf(d.x), fabsf(d.y)), fmaxf(fabsf(d.z), fabsf(d.w)))));
    }
    ss = warp_sum(ss);
    xm = warp_max(xm);
    if (lane == 0) {
      sh_ss1[warp] = ss;
      sh_xm1[warp] = xm;
    }
    __syncthreads();
    float tot = 0.f, xmx = 0.f;
    unsigned wmx = 0u;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) {
      tot += sh_ss1[w];
      xmx = fmaxf(xmx, sh_xm1[w]);
      wmx = max(wmx, sh_wmax[w]);
    }
    const float rs = rsqrtf(tot * (1.0f / (float)p.K) + p.eps);
    const float bound = xmx * __half2float(__ushort_as_half((unsigned short)wmx)) * rs * 1.002f;  // >= every |x * rs * w|
    int E = ((__float_as_int(bound) >> 23) & 255) - 112;  // fp16 biased exponent of the bound: |x| < 2^(E - 14)
    if (E < 1) E = 1;
    if (E > 30) E = 30;
    const int e = 29 - E;
    const float f = __int_as_float((127 + e) << 23), g = f * 0.0625f;
    if (threadIdx.x == 0) sh_back[0] = __int_as_float((127 + 24 - e) << 23);
    const float2 w0 = __half22float2(u2h2(nw_slice.x)), w1 = __half22float2(u2h2(nw_slice.y)), w2 = __half22float2(u2h2(nw_slice.z)),
                 w3 = __half22float2(u2h2(nw_slice.w));
    // normalised activations rounded to fp16 first (that is the operator's input), then scaled
    const float2 o0 = __half22float2(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
    const float2 o1 = __half22float2(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
    const float2 o2 = __half22float2(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
    const float2 o3 = __half22float2(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
    float sx = valid ? ((o0.x + o0.y) + (o1.x + o1.y) + (o2.x + o2.y) + (o3.x + o3.y)) * f : 0.f;
    sx += __shfl_xor_sync(0xffffffffu, sx, 1);
    sx += __shfl_xor_sync(0xffffffffu, sx, 2);
    if (valid) {
      // natural order (x0,x1)(x2,x3)(x4,x5)(x6,x7) -> (x0,x4)(x1,x5)(x2,x6)(x3,x7); odd k meet high nibbles
      uint4 q;
      q.x = h22u(__floats2half2_rn(o0.x * f, o2.x * f));
      q.y = h22u(__floats2half2_rn(o0.y * g, o2.y * g));
      q.z = h22u(__floats2half2_rn(o1.x * f, o3.x * f));
      q.w = h22u(__floats2half2_rn(o1.y * g, o3.y * g));
      *reinterpret_cast<uint4 *>(xs + threadIdx.x * 8) = q;
      if ((threadIdx.x & 3) == 0) corr[threadIdx.x >> 2] = sx * (8.0f * 5.9604644775390625e-8f);
    }
  } else {
  unsigned mx[M];
#pragma unroll
  for (int m = 0; m < M; ++m) mx[m] = 0u;
  auto track = [&](uint4 v, int m) {
    const unsigned a = (v.x & 0x7FFF7FFFu), b = (v.y & 0x7FFF7FFFu), c = (v.z & 0x7FFF7FFFu), d = (v.w & 0x7FFF7FFFu);
    unsigned t = max(max(a & 0xFFFFu, a >> 16), max(b & 0xFFFFu, b >> 16));
    t = max(t, max(max(c & 0xFFFFu, c >> 16), max(d & 0xFFFFu, d >> 16)));
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
      if (mm == m) mx[mm] = max(mx[mm], t);
  };
  if (PRO == PRO_PLAIN) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < M * rows; i += GEMV_THREADS) {
      const int m = i / rows, r = i % rows;
      const uint4 v = *reinterpret_cast<const uint4 *>(xg + (size_t)m * p.K + k_begin + r * 8);
      track(v, m);
      *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = permute(v);
    }
  } else if (PRO == PRO_SILU_MUL) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < M * rows; i += GEMV_THREADS) {
      const int m = i / rows, r = i % rows;
      const uint4 gv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * p.K + k_begin + r * 8);
      const uint4 uv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * p.K + p.K + k_begin + r * 8);
      const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
        o[j] = h22u(__floats2half2_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x, __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y));
      }
      const uint4 v = make_uint4(o[0], o[1], o[2], o[3]);
      track(v, m);
      *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = permute(v);
    }
  } else {
    __shared__ float sh_ss[GEMV_WARPS];
    const float *xg = reinterpret_cast<const float *>(p.x);
    const int rowsK = p.K / 8;
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int r = threadIdx.x; r < rowsK; r += GEMV_THREADS) {
        const float4 a = *reinterpret_cast<const float4 *>(xg + (size_t)m * p.K + r * 8);
        const float4 b = *reinterpret_cast<const float4 *>(xg + (size_t)m * p.K + r * 8 + 4);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) sh_ss[warp] = ss;
      __syncthreads();
      float tot = (lane < GEMV_WARPS) ? sh_ss[lane] : 0.f;
      tot = warp_sum(tot);
      __syncthreads();
      const float rs = rsqrtf(tot * (1.0f / (float)p.K) + p.eps);
      for (int r = threadIdx.x; r < rows; r += GEMV_THREADS) {
        const float *xr = xg + (size_t)m * p.K + k_begin + r * 8;
        const float4 a = *reinterpret_cast<const float4 *>(xr), b = *reinterpret_cast<const float4 *>(xr + 4);
        const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + k_begin + r * 8);
        const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)),
                     w3 = __half22float2(u2h2(wv.w));
        uint4 o;
        o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
        o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
        o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
        o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
        track(o, m);
        *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = permute(o);
      }
    }
  }
  // largest |x| bit pattern per batch row -> exponent e
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const unsigned wm = __reduce_max_sync(0xffffffffu, mx[m]);
    if (lane == 0) sh_max[m][warp] = wm;
  }
  __syncthreads();
  float up[M];  // 2^e
#pragma unroll
  for (int m = 0; m < M; ++m) {
    unsigned t = 0u;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) t = max(t, sh_max[m][w]);
    int E = (int)(t >> 10);          // biased fp16 exponent of the largest magnitude: |x| < 2^(E - 14)
    if (E < 1) E = 1;                // all zero or subnormal
    if (E > 30) E = 30;              // inf/nan rows: no scaling that helps
    const int e = 29 - E;            // |x| * 2^e < 2^15
    up[m] = __int_as_float((127 + e) << 23);
    if (threadIdx.x == 0) sh_back[m] = __int_as_float((127 + 24 - e) << 23);
  }
  // second pass over the same elements (each thread rescales what it staged): x * 2^e, the
  // high-nibble words another 1/16, and the per-unit sums (4 packed rows = 4 adjacent lanes)
  {
    const int n_pad = (M * rows + 31) & ~31;
    for (int i = threadIdx.x; i < n_pad; i += GEMV_THREADS) {
      const bool valid = i < M * rows;
      const int m = valid ? i / rows : 0, r = valid ? i % rows : 0;
      float f = 0.f;
#pragma unroll
      for (int mm = 0; mm < M; ++mm)
        if (mm == m) f = up[mm];
      uint4 *slot = reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8);
      float sx = 0.f;
      if (valid) {
        const uint4 v = *slot;
        const float2 a = __half22float2(u2h2(v.x)), b = __half22float2(u2h2(v.y)), c = __half22float2(u2h2(v.z)), d = __half22float2(u2h2(v.w));
        const float g = f * 0.0625f;
        sx = ((a.x + a.y) + (b.x + b.y) + (c.x + c.y) + (d.x + d.y)) * f;
        uint4 o;
        o.x = h22u(__floats2half2_rn(a.x * f, a.y * f));
        o.y = h22u(__floats2half2_rn(b.x * g, b.y * g));
        o.z = h22u(__floats2half2_rn(c.x * f, c.y * f));
        o.w = h22u(__floats2half2_rn(d.x * g, d.y * g));
        *slot = o;
      }
      sx += __shfl_xor_sync(0xffffffffu, sx, 1);
      sx += __shfl_xor_sync(0xffffffffu, sx, 2);
      if (valid && (r & 3) == 0) corr[m * n_units + (r >> 2)] = sx * (8.0f * 5.9604644775390625e-8f);
    }
  }
  }  // general prologue
  __syncthreads();

  float facc[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) facc[m][c] = 0.f;

  const uint4 *xp = reinterpret_cast<const uint4 *>(xs) + warp * UNIT_ROWS;  // this warp's unit within the slice
  const unsigned xm_step = (unsigned)xs_stride / 8;                            // uint4 elements between batch rows
  const float *cp = corr + warp;                                               // this warp's unit correction
  auto compute_unit = [&](int b) {
    constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
    __half2 hacc[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) hacc[m][c] = u2h2(0u);
#pragma unroll
    for (int r = 0; r < UNIT_ROWS; ++r) {
      uint4 xr[M];
#pragma unroll
      for (int m = 0; m < M; ++m) xr[m] = xp[m * xm_step + r];
      const uint32_t wr[4] = {wbuf[b][r].x, wbuf[b][r].y, wbuf[b][r].z, wbuf[b][r].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t w = wr[c], w8 = w >> 8;
        const __half2 v0 = u2h2(w & LO), v1 = u2h2(w & HI), v2 = u2h2(w8 & LO), v3 = u2h2(w8 & HI);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          hacc[m][c] = __hfma2(v0, u2h2(xr[m].x), hacc[m][c]);
          hacc[m][c] = __hfma2(v1, u2h2(xr[m].y), hacc[m][c]);
          hacc[m][c] = __hfma2(v2, u2h2(xr[m].z), hacc[m][c]);
          hacc[m][c] = __hfma2(v3, u2h2(xr[m].w), hacc[m][c]);
        }
      }
    }
    const float2 s01 = __half22float2(u2h2(sbuf[b].x)), s23 = __half22float2(u2h2(sbuf[b].y));
    const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float zp = cp[m * n_units];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = __half22float2(hacc[m][c]);
        facc[m][c] = fmaf(sc[c], (f.x + f.y) - zp, facc[m][c]);
      }
    }
    xp += UNIT_ROWS * GEMV_WARPS;
    cp += GEMV_WARPS;
  };

  // NBUF-deep software pipeline over this warp's units: a buffer is refilled as soon as it is consumed.
  while (u < u_end) {
#pragma unroll
    for (int b = 0; b < NBUF; ++b) {
      if (u < u_end) {
        compute_unit(b);
        if (u_load < u_end) load_unit(b);
      }
      u += GEMV_WARPS;
    }
  }

  if (p.pdl_late) pdl_launch_dependents();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float back = sh_back[m];
#pragma unroll
    for (int c = 0; c < 4; ++c) facc[m][c] *= back;
  }
  reduce_and_store<M, EPI, GEMV_THREADS, GEMV_WARPS>(facc, red, part, p.out, p.N, tile * TILE_N);
}

// fp32 activations / scales / result: the dtypes the in-tree sample declares
// (samples/05_llama2_7b_int4.py:75,133,139).  w = scale * (q - 8) is one fp32 multiply, as in
// IR statement 2; products accumulate in fp32.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS) w4a16_gemv_f32_kernel(GemvParams p) {
  pdl_launch_dependents();
  pdl_wait();  // this variant has no preamble worth overlapping: wait first
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  if (cs > 1) cluster_arrive_started();
  const int tile = blockIdx.x / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = tile * TILE_N + lane * 4;
  const bool col_ok = n0 < p.N;
  const int u_begin = (int)((long)p.units * krank / cs), u_end = (int)((long)p.units * (krank + 1) / cs);
  const int k_begin = u_begin * UNIT_K, kslice = (u_end - u_begin) * UNIT_K;

  const int xs_stride = p.xs_stride;
  float *xs = reinterpret_cast<float *>(smem_raw);
  float *red = xs + (size_t)M * xs_stride;
  float *part = red + GEMV_WARPS * M * TILE_N;

  const float *xg = reinterpret_cast<const float *>(p.x);
  for (int i = threadIdx.x; i < M * (kslice / 4); i += GEMV_THREADS) {
    const int m = i / (kslice / 4), r = i % (kslice / 4);
    *reinterpret_cast<float4 *>(xs + (size_t)m * xs_stride + r * 4) =
        *reinterpret_cast<const float4 *>(xg + (size_t)m * p.K + k_begin + r * 4);
  }
  __syncthreads();

  float facc[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) facc[m][c] = 0.f;

  const int32_t *qcol = p.qw + n0;
  const float *scol = reinterpret_cast<const float *>(p.scales) + n0;
  for (int u = u_begin + warp; u < u_end && col_ok; u += GEMV_WARPS) {
    uint4 wv[UNIT_ROWS];
    const int32_t *q = qcol + (size_t)u * UNIT_ROWS * p.N;
#pragma unroll
    for (int r = 0; r < UNIT_ROWS; ++r) wv[r] = ldg_stream_v4(q + (size_t)r * p.N);
    const float4 s4 = *reinterpret_cast<const float4 *>(scol + (size_t)((u * UNIT_K) / p.group) * p.N);
    const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
    const float *xu = xs + (u - u_begin) * UNIT_K;
#pragma unroll
    for (int r = 0; r < UNIT_ROWS; ++r) {
      const uint32_t wr[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xv[M];
#pragma unroll
        for (int m = 0; m < M; ++m) xv[m] = xu[(size_t)m * xs_stride + r * 8 + j];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          // 2^23 + q as a float, minus (2^23 + 8): q - 8 exactly.
          const float qm8 = __uint_as_float(0x4B000000u | ((wr[c] >> (4 * j)) & 15u)) - 8388616.0f;
          const float w = sc[c] * qm8;
#pragma unroll
          for (int m = 0; m < M; ++m) facc[m][c] = fmaf(xv[m], w, facc[m][c]);
        }
      }
    }
  }
  reduce_and_store<M, EPI_STORE_F32, GEMV_THREADS, GEMV_WARPS>(facc, red, part, p.out, p.N, tile * TILE_N);
}

// ---- host side -------------------------------------------------------------------------------

static int pick_cluster(int tiles, int units) {
  if (gemv_tuning_cluster() > 0) return gemv_tuning_cluster();
  const int target = 2 * sm_count();
  int cs = 1;
  while (cs < 8 && tiles * cs < target && units / (cs * 2) >= GEMV_WARPS) cs *= 2;
  return cs;
}

template <typename Kern>
static int launch_gemv(Kern kern, GemvParams p, int M, int elt, cudaStream_t stream) {
  const int tiles = (p.N + TILE_N - 1) / TILE_N;
  const int cs = pick_cluster(tiles, p.units);
  const int kslice_max = ((p.units + cs - 1) / cs) * UNIT_K;
  p.xs_stride = kslice_max;
  p.pdl_late = pdl_mode() == 2;
  size_t smem = (((size_t)M * kslice_max * elt + 15) & ~(size_t)15) +
                (size_t)(GEMV_WARPS + 1) * M * TILE_N * sizeof(float) + (size_t)M * (kslice_max / UNIT_K) * sizeof(float);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: K slice of %d values x M=%d does not fit shared memory", kslice_max, M);
  // Raising the limit is idempotent; doing it per launch keeps the library stateless across devices.
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * cs, 1, 1);
  cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
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

static int check_gemv_args(const void *x, const int32_t *qw, const void *scales, const void *out, int M,
                           int K, int N, int group) {
  AB200_REQUIRE(x && qw && scales && out, "w4a16_gemv: null pointer");
  AB200_REQUIRE(M >= 1 && M <= 16, "w4a16_gemv: M=%d outside 1..16 (use ab200_w4a16_gemm for prefill)", M);
  AB200_REQUIRE(K > 0 && K % UNIT_K == 0, "w4a16_gemv: K=%d must be a positive multiple of 32", K);
  AB200_REQUIRE(group > 0 && group % UNIT_K == 0 && K % group == 0, "w4a16_gemv: group=%d must be a multiple of 32 dividing K=%d", group, K);
  AB200_REQUIRE(N > 0 && N % 4 == 0, "w4a16_gemv: N=%d must be a positive multiple of 4", N);
  AB200_REQUIRE(aligned16(x) && aligned16(qw) && aligned16(scales) && aligned16(out), "w4a16_gemv: pointers must be 16-byte aligned");
  return AB200_OK;
}

template <int EPI, int PRO>
static int gemv_f16_direct(GemvParams p, int M, cudaStream_t s) {
  // Batches above 4 re-stream the weights per group of 4 rows.
  const size_t out_elt = (EPI == EPI_STORE) ? sizeof(__half) : sizeof(float);
  const size_t x_row_bytes = (PRO == PRO_RMSNORM) ? (size_t)p.K * 4 : (PRO == PRO_SILU_MUL) ? (size_t)p.K * 4 : (size_t)p.K * 2;
  for (int m0 = 0; m0 < M; m0 += 4) {
    const int mc = (M - m0 < 4) ? (M - m0) : 4;
    GemvParams q = p;
    q.x = reinterpret_cast<const char *>(p.x) + (size_t)m0 * x_row_bytes;
    q.out = reinterpret_cast<char *>(p.out) + (size_t)m0 * p.N * out_elt;
    int rc;
    switch (mc) {
      case 1: rc = launch_gemv(w4a16_gemv_f16_kernel<1, EPI, PRO>, q, 1, 2, s); break;
      case 2: rc = launch_gemv(w4a16_gemv_f16_kernel<2, EPI, PRO>, q, 2, 2, s); break;
      case 3: rc = launch_gemv(w4a16_gemv_f16_kernel<3, EPI, PRO>, q, 3, 2, s); break;
      default: rc = launch_gemv(w4a16_gemv_f16_kernel<4, EPI, PRO>, q, 4, 2, s); break;
    }
    if (rc) return rc;
  }
  return AB200_OK;
}

// Library-owned scratch for the persistent kernel's K-slice partials and tile counters (all of it zeroed when allocated)
static int library_scratch(size_t bytes, void **out) {
  const size_t want = bytes < ((size_t)8 << 20) ? ((size_t)8 << 20) : bytes;
  return library_buffer(LIB_BUF_PERSIST, bytes, want, want, out);
}

template <int PRO>
static int gemv_f16_scalar(GemvParams p, int M, int epi, cudaStream_t s) {
  if (epi == EPI_STORE) return gemv_f16_direct<EPI_STORE, PRO>(p, M, s);
  if (epi == EPI_RESIDUAL) return gemv_f16_direct<EPI_RESIDUAL, PRO>(p, M, s);
  return gemv_f16_direct<EPI_STORE_F32, PRO>(p, M, s);
}

// fp16 path.  Auto choice (measured on B200): one row on the scalar-pipe cluster kernel (lowest
// fixed cost and best streaming rate at that size); 2-16 rows on the TMA-ring warp-MMA kernels
// (activations resident in shared memory, or streamed through the ring for wide projections at
// 5-16 rows) when the shape fits them (group 128, N % 8 == 0), else
// 3-16 rows on the cluster warp-MMA kernel, else the scalar-pipe kernel.  The persistent warp-MMA kernel (option gemv_impl=3)
// needs scratch; scratch == nullptr means the library-owned buffer.
// One-shot prefetch hint of the calling thread (ab200_w4a16_gemv_prefetch_hint): consumed by the
// next fp16 GEMV call, whichever kernel it picks (only the scalar-pipe kernel acts on it).
static thread_local const unsigned char *t_hint_ptr[2] = {nullptr, nullptr};
static thread_local unsigned t_hint_bytes[2] = {0, 0};

static int gemv_f16_impl(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                         int K, int N, int group, int epi, void *scratch, cudaStream_t s);
static int gemv_f16(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                    int K, int N, int group, int epi, void *scratch, cudaStream_t s) {
  const int rc = gemv_f16_impl(x, pro, norm_w, eps, qw, scales, out, M, K, N, group, epi, scratch, s);
  t_hint_ptr[0] = t_hint_ptr[1] = nullptr;
  t_hint_bytes[0] = t_hint_bytes[1] = 0;
  return rc;
}

static int gemv_f16_impl(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                    int K, int N, int group, int epi, void *scratch, cudaStream_t s) {
  const int impl = gemv_tuning_impl();
  const bool persist_ok = gemv_persist_fits(M, K, N) && N % 4 == 0;
  if (impl == 3 && persist_ok) {
    if (!scratch) {
      if (int rc = library_scratch(gemv_persist_scratch_bytes(M, K, N), &scratch)) return rc;
    }
    return gemv_persist_dispatch(x, norm_w, eps, qw, scales, out, M, K, N, group, pro, epi, scratch, s);
  }
  if (impl == 5 && gemv_ring_eligible(M, K, N, group, false))
    return gemv_ring_dispatch(x, pro, norm_w, eps, qw, scales, out, K, N, epi, false, s);
  if (impl == 7) {
    bool handled = false;
    const int rc = gemv_tc_dispatch(x, pro, norm_w, eps, qw, scales, out, M, K, N, group, epi, s, &handled);
    if (rc || handled) return rc;
  }
  // streamed activations: measured faster than the resident-activation TMA kernel for wide projections at 9-16
  // rows (gate|up at 16 rows: 20 us against 33) and for the widest at 5-8 rows
  if (impl == 6 || (impl == 0 && ((M >= 9 && N >= 8192) || (M >= 5 && N >= 16384)))) {
    bool handled = false;
    // a caller's workspace holds the slabs behind the persistent kernel's counters (which stay untouched)
    void *slabs = scratch ? reinterpret_cast<unsigned char *>(scratch) + PERSIST_COUNTER_BYTES : nullptr;
    const int rc = gemv_slab_dispatch(x, pro, norm_w, eps, qw, scales, out, M, K, N, group, epi, slabs, s, &handled);
    if (rc || handled) return rc;
  }
  if (impl == 4 || (impl == 0 && M >= 2)) {
    bool handled = false;
    const int rc = gemv_tma_dispatch(x, pro, norm_w, eps, qw, scales, out, M, K, N, group, epi, s, &handled);
    if (rc || handled) return rc;
  }
  if ((impl == 2 || (impl == 0 && M > 2)) && gemv_mma_eligible(AB200_F16, M, K, N))
    return gemv_mma_dispatch(x, pro, norm_w, eps, qw, scales, out, M, K, N, group, epi, s);
  GemvParams p{x, qw, scales, out, K, N, group, K / UNIT_K, 0};
  p.norm_w = norm_w;
  p.eps = eps;
  for (int r = 0; r < 2; ++r) {
    p.pf[r] = t_hint_ptr[r];
    p.pf_bytes[r] = t_hint_bytes[r];
  }
  if (pro == PRO_PLAIN) return gemv_f16_scalar<PRO_PLAIN>(p, M, epi, s);
  if (pro == PRO_RMSNORM) return gemv_f16_scalar<PRO_RMSNORM>(p, M, epi, s);
  return gemv_f16_scalar<PRO_SILU_MUL>(p, M, epi, s);
}

}  // namespace ab200
extern "C" int ab200_w4a16_gemv_prefetch_hint(const void *p0, size_t bytes0, const void *p1, size_t bytes1) {
  using namespace ab200;
  clear_error();
  AB200_REQUIRE((!p0 || aligned16(p0)) && (!p1 || aligned16(p1)), "gemv_prefetch_hint: pointers must be 16-byte aligned");
  AB200_REQUIRE(bytes0 < (1ull << 32) && bytes1 < (1ull << 32), "gemv_prefetch_hint: ranges are limited to 4 GiB");
  t_hint_ptr[0] = reinterpret_cast<const unsigned char *>(p0);
  t_hint_ptr[1] = reinterpret_cast<const unsigned char *>(p1);
  t_hint_bytes[0] = p0 ? (unsigned)bytes0 : 0;
  t_hint_bytes[1] = p1 ? (unsigned)bytes1 : 0;
  return AB200_OK;
}
namespace ab200 {

static int gemv_f32_dispatch(GemvParams p, int M, cudaStream_t s) {
  for (int m0 = 0; m0 < M; m0 += 2) {
    const int mc = (M - m0 < 2) ? (M - m0) : 2;
    GemvParams q = p;
    q.x = reinterpret_cast<const float *>(p.x) + (size_t)m0 * p.K;
    q.out = reinterpret_cast<float *>(p.out) + (size_t)m0 * p.N;
    int rc = (mc == 1) ? launch_gemv(w4a16_gemv_f32_kernel<1>, q, 1, 4, s)
                       : launch_gemv(w4a16_gemv_f32_kernel<2>, q, 2, 4, s);
    if (rc) return rc;
  }
  return AB200_OK;
}

// x_f32[i] += fp16_round(partial_f32[i]): the residual update after a tensor-parallel all-reduce.
__global__ void residual_add_kernel(float *__restrict__ x, const float *__restrict__ partial, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    x[i] += __half2float(__float2half_rn(partial[i]));
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_w4a16_gemv(const void *x, const int32_t *qweight, const void *scales, void *out,
                                int M, int K, int N, int group, int dtype, void *stream) {
  clear_error();
  if (int rc = check_gemv_args(x, qweight, scales, out, M, K, N, group)) return rc;
  if (dtype == AB200_F16) return gemv_f16(x, PRO_PLAIN, nullptr, 0.f, qweight, scales, out, M, K, N, group, EPI_STORE, nullptr, (cudaStream_t)stream);
  if (dtype == AB200_F32) {
    GemvParams p{x, qweight, scales, out, K, N, group, K / UNIT_K, 0};
    return gemv_f32_dispatch(p, M, (cudaStream_t)stream);
  }
  return fail(AB200_EINVAL, "w4a16_gemv: unknown dtype %d", dtype);
}

extern "C" int ab200_w4a16_gemv_residual(const void *x, const int32_t *qweight, const void *scales,
                                         float *resid_f32, int M, int K, int N, int group, void *stream) {
  clear_error();
  if (int rc = check_gemv_args(x, qweight, scales, resid_f32, M, K, N, group)) return rc;
  return gemv_f16(x, PRO_PLAIN, nullptr, 0.f, qweight, scales, resid_f32, M, K, N, group, EPI_RESIDUAL, nullptr, (cudaStream_t)stream);
}

extern "C" int ab200_w4a16_gemv_f32out(const void *x, const int32_t *qweight, const void *scales,
                                       float *out_f32, int M, int K, int N, int group, void *stream) {
  clear_error();
  if (int rc = check_gemv_args(x, qweight, scales, out_f32, M, K, N, group)) return rc;
  return gemv_f16(x, PRO_PLAIN, nullptr, 0.f, qweight, scales, out_f32, M, K, N, group, EPI_STORE_F32, nullptr, (cudaStream_t)stream);
}

static size_t gemv_workspace_bytes(int M, int K, int N) {
  const size_t a = gemv_persist_scratch_bytes(M, K, N), b = PERSIST_COUNTER_BYTES + gemv_slab_scratch_bytes(M, K);
  return a > b ? a : b;
}
extern "C" size_t ab200_w4a16_gemv_workspace_bytes(int M, int K, int N) {
  return gemv_workspace_bytes(M, K, N);
}

extern "C" int ab200_w4a16_gemv_fused(const void *x, int prologue, const void *norm_weight_f16, float eps, const int32_t *qweight,
                                      const void *scales, void *out, int epilogue, int M, int K, int N, int group,
                                      void *workspace, size_t workspace_bytes, void *stream) {
  clear_error();
  if (int rc = check_gemv_args(x, qweight, scales, out, M, K, N, group)) return rc;
  AB200_REQUIRE(prologue >= 0 && prologue <= 2 && epilogue >= 0 && epilogue <= 2, "w4a16_gemv_fused: bad prologue %d / epilogue %d", prologue, epilogue);
  AB200_REQUIRE(prologue != PRO_RMSNORM || norm_weight_f16 != nullptr, "w4a16_gemv_fused: RMSNorm prologue needs a weight vector");
  AB200_REQUIRE(workspace == nullptr || (aligned16(workspace) && workspace_bytes >= gemv_workspace_bytes(M, K, N)),
                "w4a16_gemv_fused: workspace must be 16-byte aligned and hold %zu bytes", gemv_workspace_bytes(M, K, N));
  return gemv_f16(x, prologue, reinterpret_cast<const __half *>(norm_weight_f16), eps, qweight, scales, out, M, K, N, group, epilogue,
                  workspace, (cudaStream_t)stream);
}

extern "C" int ab200_w4a16_gemv_tiled(const void *x, int prologue, const void *norm_weight_f16, float eps, const int32_t *qweight_tiled,
                                      const void *scales_tiled, void *out, int epilogue, int M, int K, int N, int group, void *stream) {
  clear_error();
  if (int rc = check_gemv_args(x, qweight_tiled, scales_tiled, out, M, K, N, group)) return rc;
  AB200_REQUIRE(prologue >= 0 && prologue <= 2 && epilogue >= 0 && epilogue <= 2, "w4a16_gemv_tiled: bad prologue %d / epilogue %d", prologue, epilogue);
  AB200_REQUIRE(prologue != PRO_RMSNORM || norm_weight_f16 != nullptr, "w4a16_gemv_tiled: RMSNorm prologue needs a weight vector");
  AB200_REQUIRE(N % TILE_N == 0, "w4a16_gemv_tiled: N=%d must be a multiple of %d for the tile-major layout", N, TILE_N);
  AB200_REQUIRE(M <= 4, "w4a16_gemv_tiled: batch %d (the tile-major path serves batches of 1-4 rows)", M);
  {
    const int impl = gemv_tuning_impl();
    // the bulk-copy ring kernel on request; in a decode step (a chain of dependent kernels) it runs level with
    // the register-prefetch kernel, whose smaller footprint lets the next kernel's CTAs become resident earlier
    if (impl == 5 && gemv_ring_eligible(M, K, N, group, true))
      return gemv_ring_dispatch(x, prologue, reinterpret_cast<const __half *>(norm_weight_f16), eps, qweight_tiled, scales_tiled, out, K, N,
                                epilogue, true, (cudaStream_t)stream);
  }
  GemvParams p{x, qweight_tiled, scales_tiled, out, K, N, group, K / UNIT_K, 0};
  p.norm_w = reinterpret_cast<const __half *>(norm_weight_f16);
  p.eps = eps;
  p.ld_w = TILE_N;
  p.ld_s = TILE_N;
  p.tile_w = (size_t)(K / 8) * TILE_N;
  p.tile_s = (size_t)(K / group) * TILE_N;
  if (prologue == PRO_PLAIN) return gemv_f16_scalar<PRO_PLAIN>(p, M, epilogue, (cudaStream_t)stream);
  if (prologue == PRO_RMSNORM) return gemv_f16_scalar<PRO_RMSNORM>(p, M, epilogue, (cudaStream_t)stream);
  return gemv_f16_scalar<PRO_SILU_MUL>(p, M, epilogue, (cudaStream_t)stream);
}

extern "C" int ab200_residual_add(float *x_f32, const float *partial_f32, int n, void *stream) {
  clear_error();
  AB200_REQUIRE(x_f32 && partial_f32 && n > 0, "residual_add: bad argument");
  residual_add_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(x_f32, partial_f32, n);
  AB200_CHECK_LAUNCH("residual_add");
  return AB200_OK;
}

extern "C" int ab200_set_option(const char *name, int value) {
  clear_error();
  AB200_REQUIRE(name != nullptr, "set_option: null name");
  return gemv_tuning_set(name, value);
}

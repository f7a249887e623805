// W4A16 decode GEMV, bulk-copy ring variant (batch 1, fp16 activations/scales, group 128).
//
// Replaces the kernel the reference generates from samples/05_llama2_7b_int4.py:135-139 for the
// decode step's one-row projections.
//
// The register-prefetch kernel (w4a16_gemv.cu) keeps at most 2 x 64 B per thread in flight, so its
// warps stall on their own global loads and HBM idles at every kernel boundary.  Here the bytes in
// flight do not depend on what the warps are doing: one producer thread per CTA keeps a ring of
// DEPTH shared-memory stages full with bulk copies (`cp.async.bulk`, completion on an mbarrier).
// A stage is one quantisation group of a column tile: 16 packed rows x 128 columns = 8 KiB.
//   * tile-major weights ([N/128][K/8][128], what the decoder keeps in HBM): the stages of a CTA
//     are one contiguous byte range, one 8 KiB linear bulk copy per stage;
//   * reference layout ([K/8, N]): one tensor-map copy of a 128-column x 16-row box per stage,
//     which lands in shared memory in exactly the same [16][128] order.
// The copies of the first DEPTH stages and of the slice's scale rows are issued before
// `griddepcontrol.wait`: weights never depend on the kernel before, so with programmatic
// dependent launch they stream while the predecessor is still in its tail and while this
// kernel's activations are being staged.
//
// Eight consumer warps in four pairs: stage s belongs to pair s & 3, and the pair's two warps take
// packed rows 0-7 and 8-15 of it: eight conflict-free 16-byte shared loads per thread (lane l reads
// columns 4l..4l+3), 32 packed words per visit, then the raw-nibble multiply of the scalar kernel: `w & 0x000F000F` is a pair
// of fp16 subnormals q * 2^-24 (`w & 0x00F000F0` = 16 q * 2^-24), multiplied on the FP16 pipe by
// activations pre-scaled by a power of two, 16 products per half2 lane, widened to fp32, zero-point
// removed as 8 * sum(x) per 32-k unit, times the group scale.  A warp hands its part of a stage
// back (mbarrier arrive) as soon as the packed words are in registers.
//
// Split-K: the stage ranges of one column tile are the CTAs of a thread-block cluster; sums meet
// in the owner CTA's inbox through distributed shared memory (a split cluster barrier: arrive at
// kernel start, wait before the first remote store, so a peer CTA is known to be running before
// its shared memory is written), fixed order, bitwise repeatable, no scratch, no atomics.
//
// Tensor-parallel row-parallel projections (epilogue EPI_ALLREDUCE) fuse the sum over ranks into
// the same kernel: the thread that owns an output column pushes its fp32 sum as an 8-byte
// (value, epoch) pair straight into slot `rank` of every peer's receive buffer (plain peer stores
// over NVLink, no multicast, the buffers of comm.cu), then polls its OWN buffer for the same column
// from the other ranks (bounded), adds the contributions in rank order (bit-identical on every
// rank) and applies x += fp16_round(sum).  All column tiles exchange at once from as many SMs as
// the projection uses, and the separate all-reduce kernel disappears.  The exchange number comes
// from the buffer's epoch word: every CTA reads it, then takes a ticket; the CTA that draws the
// last ticket advances the epoch for the next exchange.
//
// Every wait is bounded; a wait that runs out stores a site code in the status word
// (ab200_kernel_status: 400 + slot producer, 410 + slot consumer, 420 scales, 100 + peer for the
// exchange) and the kernel finishes with whatever it has.  An exchange that finds the status word
// already set polls once instead of waiting (a timeout is sticky until the host reads it).
#include <cooperative_groups.h>
#include <cuda.h>  // CUtensorMap (types only)

#include "common.cuh"
#include "gemv_shared.cuh"

namespace cg = cooperative_groups;

namespace ab200 {

constexpr int R_CWARPS = 8;                      // consumer warps: 2 groups x 4
constexpr int R_CTHREADS = R_CWARPS * 32;
constexpr int R_THREADS = R_CTHREADS + 32;       // + the producer warp
constexpr int R_STAGE_ROWS = 16;                 // packed rows per stage = one 128-k group
constexpr int R_STAGE_BYTES = R_STAGE_ROWS * TILE_N * 4;  // 8 KiB
constexpr int R_SCALE_ROW_BYTES = TILE_N * 2;    // one group's scales for the tile
constexpr int R_MAX_DEPTH = 16;
constexpr int R_MAX_WORLD = 8;
constexpr int EPI_ALLREDUCE = 3;  // x_f32 += fp16_round(sum over ranks): fused push all-reduce

struct RingParams {
  const void *x;
  const __half *norm_w;
  const int32_t *qw;
  const __half *scales;
  void *out;
  int *status;
  int K, N;
  int groups;   // K / 128 = stages per column tile
  int depth;    // ring stages (a multiple of 4)
  int tiled;    // 1: tile-major weights, linear bulk copies; 0: reference layout, tensor-map copies
  int pdl_late;
  float eps;
  unsigned wait_polls;
  // EPI_ALLREDUCE: every rank's receive buffer as mapped here (layout of comm.cu:
  // uint2 slots[2][world][n_max]; int epoch; int ticket), own entry = local memory
  uint2 *slots[R_MAX_WORLD];
  int *epoch;
  int rank, world, n_max;
  unsigned comm_polls;
};

__device__ __forceinline__ uint32_t r_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool r_mbar_wait(uint32_t bar, unsigned parity, unsigned polls) {
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

// Out of the streaming loop's way: entered only when the first try did not succeed.
__device__ __noinline__ bool r_mbar_wait_slow(uint32_t bar, unsigned parity, unsigned polls) { return r_mbar_wait(bar, parity, polls); }

__device__ __forceinline__ void r_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}

__device__ __forceinline__ void r_tma_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void r_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(R_CTHREADS) : "memory"); }

// Stages this CTA's K slice of the activation row in shared memory for the raw-nibble multiply:
// packed row r holds (x0,x4)(x1,x5)(x2,x6)(x3,x7) of its eight k-values, scaled by 2^e (the words
// that meet high nibbles by 2^(e-4)), e chosen so that the largest magnitude stays below 2^15;
// corr[u] = 8 * 2^-24 * sum over 32-k unit u of x * 2^e; *back = 2^(24 - e).  Called by the 256
// consumer threads only (its barriers are consumer barriers).
template <int PRO>
__device__ __forceinline__ void ring_stage_x(const RingParams &p, int k_begin, int rows, __half *xs, float *corr, float *back,
                                             float *sh_f, unsigned *sh_u, const uint4 *nw_pre, unsigned wmax_pre) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr float ZP = 8.0f * 5.9604644775390625e-8f;  // 8 * 2^-24
  if (PRO == PRO_RMSNORM && rows <= 2 * R_CTHREADS) {
    // one pass: the scale exponent comes from the bound max|x| * max|w| * rs, known before any
    // normalised value is
    const float *xg = reinterpret_cast<const float *>(p.x);
    float4 a[2], b[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = tid + i * R_CTHREADS;
      a[i] = b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < rows) {
        a[i] = *reinterpret_cast<const float4 *>(xg + k_begin + r * 8);
        b[i] = *reinterpret_cast<const float4 *>(xg + k_begin + r * 8 + 4);
      }
    }
    float ss = 0.f, xm = 0.f;
    for (int r = tid; r < p.K / 8; r += R_CTHREADS) {
      const float4 c = *reinterpret_cast<const float4 *>(xg + r * 8), d = *reinterpret_cast<const float4 *>(xg + r * 8 + 4);
      ss += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w + d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w;
      xm = fmaxf(fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))),
                 fmaxf(xm, fmaxf(fmaxf(fabsf(d.x), fabsf(d.y)), fmaxf(fabsf(d.z), fabsf(d.w)))));
    }
    ss = warp_sum(ss);
    xm = warp_max(xm);
    const unsigned wm = __reduce_max_sync(0xffffffffu, wmax_pre);
    if (lane == 0) {
      sh_f[warp] = ss;
      sh_f[R_CWARPS + warp] = xm;
      sh_u[warp] = wm;
    }
    r_consumer_sync();
    float tot = 0.f, xmx = 0.f;
    unsigned wmx = 0u;
#pragma unroll
    for (int w = 0; w < R_CWARPS; ++w) {
      tot += sh_f[w];
      xmx = fmaxf(xmx, sh_f[R_CWARPS + w]);
      wmx = max(wmx, sh_u[w]);
    }
    const float rs = rsqrtf(tot * (1.0f / (float)p.K) + p.eps);
    const float bound = xmx * __half2float(__ushort_as_half((unsigned short)wmx)) * rs * 1.002f;  // >= every |x * rs * w|
    int E = ((__float_as_int(bound) >> 23) & 255) - 112;  // fp16 biased exponent of the bound: |x| < 2^(E - 14)
    if (E < 1) E = 1;
    if (E > 30) E = 30;
    const int e = 29 - E;
    const float f = __int_as_float((127 + e) << 23), g = f * 0.0625f;
    if (tid == 0) *back = __int_as_float((127 + 24 - e) << 23);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = tid + i * R_CTHREADS;
      const bool valid = r < rows;
      const uint4 nw = nw_pre[i];
      const float2 w0 = __half22float2(u2h2(nw.x)), w1 = __half22float2(u2h2(nw.y)), w2 = __half22float2(u2h2(nw.z)),
                   w3 = __half22float2(u2h2(nw.w));
      // normalised activations rounded to fp16 first (that is the operator's input), then scaled
      const float2 o0 = __half22float2(__floats2half2_rn(a[i].x * rs * w0.x, a[i].y * rs * w0.y));
      const float2 o1 = __half22float2(__floats2half2_rn(a[i].z * rs * w1.x, a[i].w * rs * w1.y));
      const float2 o2 = __half22float2(__floats2half2_rn(b[i].x * rs * w2.x, b[i].y * rs * w2.y));
      const float2 o3 = __half22float2(__floats2half2_rn(b[i].z * rs * w3.x, b[i].w * rs * w3.y));
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
        *reinterpret_cast<uint4 *>(xs + r * 8) = q;
        if ((r & 3) == 0) corr[r >> 2] = sx * ZP;
      }
    }
    return;
  }

  // general route: pass 1 builds the fp16 operand row in shared memory and finds its largest
  // magnitude, pass 2 rescales what each thread staged
  unsigned mx = 0u;
  auto track = [&](uint4 v) {
    const unsigned a = (v.x & 0x7FFF7FFFu), b = (v.y & 0x7FFF7FFFu), c = (v.z & 0x7FFF7FFFu), d = (v.w & 0x7FFF7FFFu);
    unsigned t = max(max(a & 0xFFFFu, a >> 16), max(b & 0xFFFFu, b >> 16));
    t = max(t, max(max(c & 0xFFFFu, c >> 16), max(d & 0xFFFFu, d >> 16)));
    mx = max(mx, t);
  };
  if (PRO == PRO_PLAIN) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int r = tid; r < rows; r += R_CTHREADS) {
      const uint4 v = *reinterpret_cast<const uint4 *>(xg + k_begin + r * 8);
      track(v);
      *reinterpret_cast<uint4 *>(xs + r * 8) = permute_row(v);
    }
  } else if (PRO == PRO_SILU_MUL) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int r = tid; r < rows; r += R_CTHREADS) {
      const uint4 gv = *reinterpret_cast<const uint4 *>(xg + k_begin + r * 8);
      const uint4 uv = *reinterpret_cast<const uint4 *>(xg + p.K + k_begin + r * 8);
      const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
        o[j] = h22u(__floats2half2_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x, __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y));
      }
      const uint4 v = make_uint4(o[0], o[1], o[2], o[3]);
      track(v);
      *reinterpret_cast<uint4 *>(xs + r * 8) = permute_row(v);
    }
  } else {  // RMSNorm of a long slice
    const float *xg = reinterpret_cast<const float *>(p.x);
    float ss = 0.f;
    for (int r = tid; r < p.K / 8; r += R_CTHREADS) {
      const float4 a = *reinterpret_cast<const float4 *>(xg + r * 8), b = *reinterpret_cast<const float4 *>(xg + r * 8 + 4);
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) sh_f[warp] = ss;
    r_consumer_sync();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < R_CWARPS; ++w) tot += sh_f[w];
    const float rs = rsqrtf(tot * (1.0f / (float)p.K) + p.eps);
    for (int r = tid; r < rows; r += R_CTHREADS) {
      const float *xr = xg + k_begin + r * 8;
      const float4 a = *reinterpret_cast<const float4 *>(xr), b = *reinterpret_cast<const float4 *>(xr + 4);
      const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + k_begin + r * 8);
      const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)),
                   w3 = __half22float2(u2h2(wv.w));
      uint4 o;
      o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
      o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
      o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
      o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
      track(o);
      *reinterpret_cast<uint4 *>(xs + r * 8) = permute_row(o);
    }
  }
  mx = __reduce_max_sync(0xffffffffu, mx);
  if (lane == 0) sh_u[R_CWARPS + warp] = mx;
  r_consumer_sync();
  unsigned t = 0u;
#pragma unroll
  for (int w = 0; w < R_CWARPS; ++w) t = max(t, sh_u[R_CWARPS + w]);
  int E = (int)(t >> 10);  // biased fp16 exponent of the largest magnitude: |x| < 2^(E - 14)
  if (E < 1) E = 1;        // all zero or subnormal
  if (E > 30) E = 30;      // inf/nan rows: no scaling that helps
  const int e = 29 - E;    // |x| * 2^e < 2^15
  const float f = __int_as_float((127 + e) << 23), g = f * 0.0625f;
  if (tid == 0) *back = __int_as_float((127 + 24 - e) << 23);
  const int n_pad = (rows + 31) & ~31;
  for (int r = tid; r < n_pad; r += R_CTHREADS) {
    const bool valid = r < rows;
    float sx = 0.f;
    if (valid) {
      uint4 *slot = reinterpret_cast<uint4 *>(xs + r * 8);
      const uint4 v = *slot;
      const float2 a = __half22float2(u2h2(v.x)), b = __half22float2(u2h2(v.y)), c = __half22float2(u2h2(v.z)), d = __half22float2(u2h2(v.w));
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
    if (valid && (r & 3) == 0) corr[r >> 2] = sx * ZP;
  }
}

// EMU: several ranks as consecutive CTA ranges of ONE cooperative launch on one GPU (blockIdx.x /
// ctas_per_rank = rank, parameters from emu[rank]): the exchange protocol on fewer GPUs than ranks.
template <int EPI, int PRO, bool EMU>
__global__ void __launch_bounds__(R_THREADS) w4a16_gemv_ring_kernel(const __grid_constant__ CUtensorMap tm_w, const RingParams p0,
                                                                    const RingParams *__restrict__ emu, int ctas_per_rank) {
  extern __shared__ __align__(128) unsigned char r_smem[];
  __shared__ RingParams sh_p;
  int bx = blockIdx.x;
  if (EMU) {
    const int vr = blockIdx.x / ctas_per_rank;
    bx = blockIdx.x - vr * ctas_per_rank;
    if (threadIdx.x == 0) sh_p = emu[vr];
    __syncthreads();
  }
  const RingParams &p = EMU ? sh_p : p0;
  __shared__ float sh_f[2 * R_CWARPS];
  __shared__ unsigned sh_u[2 * R_CWARPS];
  __shared__ float sh_back;
  __shared__ int sh_epoch;
  __shared__ __align__(8) unsigned long long sh_bars[2 * R_MAX_DEPTH + 1];

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned cs = cluster.num_blocks(), krank = cluster.block_rank();
  const int tile = bx / cs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.depth;

  // this CTA's stages (quantisation groups) of the column tile
  const int g_begin = (int)((long)p.groups * krank / cs), g_end = (int)((long)p.groups * (krank + 1) / cs);
  const int nst = g_end - g_begin;
  const int nst_max = (p.groups + cs - 1) / cs;  // cluster-uniform: fixes the shared-memory layout
  const int k_begin = g_begin * 128, rows = nst * R_STAGE_ROWS;

  // shared memory: [ring D x 8 KiB][scales nst_max x 256 B][x nst_max x 256 B][corr nst_max x 4 floats][red 8 x 128][inbox 128]
  unsigned char *ring = r_smem;
  unsigned char *sc_s = ring + (size_t)D * R_STAGE_BYTES;
  __half *xs = reinterpret_cast<__half *>(sc_s + (size_t)nst_max * R_SCALE_ROW_BYTES);
  float *corr = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(xs) + (size_t)nst_max * 256);
  float *red = corr + nst_max * 4;
  float *part = red + R_CWARPS * TILE_N;
  const uint32_t bars = r_smem_u32(sh_bars);  // full[D], empty[D], scales
  const uint32_t bar_sc = bars + 16 * D;

  if (threadIdx.x == 0) {
    for (int i = 0; i < D; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" ::"r"(bars + 8 * (D + i)));  // the two warps that share a stage
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_sc));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // first half of the split cluster barrier: tells the peers that this CTA is running
  if (cs > 1) cluster_arrive_started();
  if (!p.pdl_late) pdl_launch_dependents();
  __syncthreads();

  float facc[4] = {0.f, 0.f, 0.f, 0.f};
  unsigned ticket = 0u;
  if (warp == R_CWARPS) {
    // ---- producer: one thread keeps the ring full; nothing here depends on the kernel before ------
    if (lane == 0 && nst > 0) {
      const unsigned char *src_w = nullptr;
      const int row0 = g_begin * R_STAGE_ROWS;
      if (p.tiled) {
        src_w = reinterpret_cast<const unsigned char *>(p.qw) + ((size_t)tile * p.groups + g_begin) * R_STAGE_BYTES;
        const unsigned char *src_s = reinterpret_cast<const unsigned char *>(p.scales) + ((size_t)tile * p.groups + g_begin) * R_SCALE_ROW_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_sc), "r"(nst * R_SCALE_ROW_BYTES) : "memory");
        r_bulk_load(r_smem_u32(sc_s), src_s, nst * R_SCALE_ROW_BYTES, bar_sc);
      } else {
        // reference layout: the tile's scale rows are 2 N bytes apart, one 256-byte copy each
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_sc), "r"(nst * R_SCALE_ROW_BYTES) : "memory");
        for (int g = 0; g < nst; ++g)
          r_bulk_load(r_smem_u32(sc_s) + g * R_SCALE_ROW_BYTES, p.scales + (size_t)(g_begin + g) * p.N + tile * TILE_N, R_SCALE_ROW_BYTES, bar_sc);
      }
      int slot = 0, round = 0;
      for (int s = 0; s < nst; ++s) {
        if (round > 0 && !r_mbar_wait(bars + 8 * (D + slot), (round - 1) & 1, p.wait_polls)) {
          atomicExch(p.status, 400 + slot);  // site 400: a ring stage was never released
          break;
        }
        const uint32_t full = bars + 8 * slot;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "n"(R_STAGE_BYTES) : "memory");
        if (p.tiled) r_bulk_load(r_smem_u32(ring) + slot * R_STAGE_BYTES, src_w + (size_t)s * R_STAGE_BYTES, R_STAGE_BYTES, full);
        else r_tma_2d(r_smem_u32(ring) + slot * R_STAGE_BYTES, &tm_w, tile * TILE_N, row0 + s * R_STAGE_ROWS, full);
        if (++slot == D) {
          slot = 0;
          ++round;
        }
      }
    }
  } else {
    // ---- consumers -------------------------------------------------------------------------------
    // what only needs the constant norm weights happens before the wait
    uint4 nw_pre[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    unsigned wmax_pre = 0u;
    if (PRO == PRO_RMSNORM && rows <= 2 * R_CTHREADS) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = threadIdx.x + i * R_CTHREADS;
        if (r < rows) nw_pre[i] = __ldg(reinterpret_cast<const uint4 *>(p.norm_w + k_begin) + r);
      }
      for (int r = threadIdx.x; r < p.K / 8; r += R_CTHREADS) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.norm_w) + r);
        const unsigned a = v.x & 0x7FFF7FFFu, b = v.y & 0x7FFF7FFFu, c = v.z & 0x7FFF7FFFu, d = v.w & 0x7FFF7FFFu;
        wmax_pre = max(wmax_pre, max(max(max(a & 0xFFFFu, a >> 16), max(b & 0xFFFFu, b >> 16)), max(max(c & 0xFFFFu, c >> 16), max(d & 0xFFFFu, d >> 16))));
      }
    }
    pdl_wait();  // x (and a residual output) may come from the kernel before this one
    if (EPI == EPI_ALLREDUCE && threadIdx.x == 0) {
      // this exchange's number, read before the ticket is taken (release): whoever draws the last
      // ticket knows that every CTA of this rank has read the epoch it is about to advance
      int *ep = p.epoch;
      sh_epoch = *reinterpret_cast<volatile int *>(ep) + 1;
      asm volatile("atom.add.release.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(ep + 1) : "memory");
    }
    ring_stage_x<PRO>(p, k_begin, rows, xs, corr, &sh_back, sh_f, sh_u, nw_pre, wmax_pre);
    r_consumer_sync();

    // Stage s belongs to warp pair s & 3; the pair's warps take packed rows 0-7 and 8-15 of it: 32 packed
    // words per thread and visit, so that the per-visit bookkeeping (wait, hand-back, pointer bumps) is
    // spread over 256 multiply-adds.  All operands come through 32-bit shared addresses.
    const int pr = warp >> 1, hf = warp & 1;
    if (nst > 0 && !r_mbar_wait(bar_sc, 0, p.wait_polls)) {
      if (lane == 0) atomicExch(p.status, 420);  // site 420: the scale rows never arrived
    }
    uint32_t w_addr = r_smem_u32(ring) + (uint32_t)(pr * R_STAGE_BYTES + hf * (R_STAGE_BYTES / 2) + lane * 16);
    const uint32_t w_end = r_smem_u32(ring) + (uint32_t)(D * R_STAGE_BYTES);
    uint32_t full_addr = bars + 8 * pr, empty_addr = bars + 8 * (D + pr);
    uint32_t x_addr = r_smem_u32(xs) + (uint32_t)((pr * R_STAGE_ROWS + hf * 8) * 16);
    uint32_t c_addr = r_smem_u32(corr) + (uint32_t)((pr * 4 + hf * 2) * 4);
    uint32_t s_addr = r_smem_u32(sc_s) + (uint32_t)(pr * R_SCALE_ROW_BYTES + lane * 8);
    unsigned parity = 0;
    constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
    // The barrier of the NEXT visit is probed (test_wait: never blocks) right after this visit's words
    // are in registers, so the probe's latency hides behind the multiply-adds; `ready` carries the
    // answer into the next round, which only enters the waiting path when the stage was not there yet.
    uint32_t ready = 0;
    if (pr < nst) asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                               : "=r"(ready) : "r"(full_addr), "r"(parity) : "memory");
    for (int s = pr; s < nst; s += 4) {
      if (!ready && !r_mbar_wait_slow(full_addr, parity, p.wait_polls)) {
        if (lane == 0) atomicExch(p.status, 410 + pr);  // site 410: a ring stage never arrived
        break;                                          // stop waiting; the result is void
      }
      uint4 wv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) wv[r] = lds128(w_addr + r * 512);
      uint2 sv, zz;
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(sv.x), "=r"(sv.y) : "r"(s_addr));
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(zz.x), "=r"(zz.y) : "r"(c_addr));
      // the packed words are in registers: hand this warp's half of the stage back
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr) : "memory");
      {  // advance to the next visit's slot and probe it
        w_addr += 4 * R_STAGE_BYTES;
        full_addr += 32;
        empty_addr += 32;
        if (w_addr >= w_end) {  // D is a multiple of 4: a slot always serves the same pair
          w_addr -= (uint32_t)(D * R_STAGE_BYTES);
          full_addr -= 8 * D;
          empty_addr -= 8 * D;
          parity ^= 1u;
        }
        ready = 0;
        if (s + 4 < nst) asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                                      : "=r"(ready) : "r"(full_addr), "r"(parity) : "memory");
      }
      {
        const float2 s01 = __half22float2(u2h2(sv.x)), s23 = __half22float2(u2h2(sv.y));
        const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          __half2 hacc[4] = {u2h2(0u), u2h2(0u), u2h2(0u), u2h2(0u)};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const uint4 xr = lds128(x_addr + (u * 4 + r) * 16);
            const uint32_t wr[4] = {wv[u * 4 + r].x, wv[u * 4 + r].y, wv[u * 4 + r].z, wv[u * 4 + r].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint32_t w = wr[c], w8 = w >> 8;
              hacc[c] = __hfma2(u2h2(w & LO), u2h2(xr.x), hacc[c]);
              hacc[c] = __hfma2(u2h2(w & HI), u2h2(xr.y), hacc[c]);
              hacc[c] = __hfma2(u2h2(w8 & LO), u2h2(xr.z), hacc[c]);
              hacc[c] = __hfma2(u2h2(w8 & HI), u2h2(xr.w), hacc[c]);
            }
          }
          const float zp = __uint_as_float(u ? zz.y : zz.x);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 f = __half22float2(hacc[c]);
            facc[c] = fmaf(sc[c], (f.x + f.y) - zp, facc[c]);
          }
        }
      }
      x_addr += 4 * R_STAGE_ROWS * 16;
      c_addr += 4 * 4 * 4;
      s_addr += 4 * R_SCALE_ROW_BYTES;
    }
    if (p.pdl_late) pdl_launch_dependents();
    const float back = sh_back;
    *reinterpret_cast<float4 *>(&red[warp * TILE_N + lane * 4]) = make_float4(facc[0] * back, facc[1] * back, facc[2] * back, facc[3] * back);
  }
  __syncthreads();

  // ---- reduction: warps -> owner CTA's inbox (push) -> cluster barrier -> rank-ordered sum -> epilogue
  const int cols_per = TILE_N / cs;
  if (cs > 1) cluster_wait_started();  // every peer CTA is running: its inbox may be written
  if (threadIdx.x < TILE_N) {
    const int c = threadIdx.x;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < R_CWARPS; ++w) s += red[w * TILE_N + c];
    const int owner = c / cols_per, cc = c - owner * cols_per;
    float *inbox = (cs > 1) ? cluster.map_shared_rank(part, owner) : part;
    inbox[krank * cols_per + cc] = s;
  }
  if (cs > 1) cluster.sync(); else __syncthreads();
  if ((int)threadIdx.x < cols_per) {
    const int cc = threadIdx.x;
    float s = 0.f;
    for (unsigned r = 0; r < cs; ++r) s += part[r * cols_per + cc];
    const int n = tile * TILE_N + krank * cols_per + cc;
    if (EPI == EPI_STORE) reinterpret_cast<__half *>(p.out)[n] = __float2half_rn(s);
    else if (EPI == EPI_STORE_F32) reinterpret_cast<float *>(p.out)[n] = s;
    else if (EPI == EPI_RESIDUAL) reinterpret_cast<float *>(p.out)[n] += __half2float(__float2half_rn(s));
    else {
      // ---- fused push all-reduce of this column over the ranks, then the residual update ----------
      const int e = sh_epoch, buf = e & 1, world = p.world, rank = p.rank;
      const unsigned tag = (unsigned)e;
      const uint32_t sbits = __float_as_uint(s);
#pragma unroll
      for (int q = 0; q < R_MAX_WORLD; ++q) {
        if (q < world && q != rank) {
          uint2 *dst = p.slots[q] + ((size_t)buf * world + rank) * p.n_max + n;
          asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1,%2};" ::"l"(dst), "r"(sbits), "r"(tag) : "memory");
        }
      }
      float v[R_MAX_WORLD];
      unsigned pending = ((1u << world) - 1u) & ~(1u << rank);
      const uint2 *mine = p.slots[rank] + (size_t)buf * world * p.n_max + n;
      const bool sticky = *reinterpret_cast<volatile int *>(p.status) != 0;
      unsigned polls = 0;
      while (pending) {
        uint2 r[R_MAX_WORLD];
#pragma unroll
        for (int q = 0; q < R_MAX_WORLD; ++q)
          if ((pending >> q) & 1u)
            asm volatile("ld.relaxed.sys.global.v2.b32 {%0,%1}, [%2];" : "=r"(r[q].x), "=r"(r[q].y) : "l"(mine + (size_t)q * p.n_max) : "memory");
#pragma unroll
        for (int q = 0; q < R_MAX_WORLD; ++q)
          if (((pending >> q) & 1u) && r[q].y == tag) {
            v[q] = __uint_as_float(r[q].x);
            pending &= ~(1u << q);
          }
        if (pending && (sticky || ++polls >= p.comm_polls)) {
          if (!sticky) atomicExch(p.status, 100 + (__ffs(pending) - 1));  // site 100 + a peer that never arrived
#pragma unroll
          for (int q = 0; q < R_MAX_WORLD; ++q)
            if ((pending >> q) & 1u) v[q] = 0.f;
          break;
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < R_MAX_WORLD; ++q)
        if (q < world) sum += (q == rank) ? s : v[q];
      reinterpret_cast<float *>(p.out)[n] += __half2float(__float2half_rn(sum));
    }
  }
  if (EPI == EPI_ALLREDUCE && threadIdx.x == 0) {
    const unsigned total = EMU ? (unsigned)ctas_per_rank : gridDim.x;
    if (ticket == total - 1) {  // every CTA of this rank has read the epoch: open the next exchange
      p.epoch[1] = 0;
      p.epoch[0] = sh_epoch;
    }
  }
}

// ---- host side -------------------------------------------------------------------------------

typedef CUresult (*RingEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int g_ring_depth = 0;             // 0 = auto

static unsigned g_ring_wait_polls = 1u << 22;

int gemv_ring_set_depth(int d) {
  if (d != 0 && (d < 4 || d > R_MAX_DEPTH || (d & 3))) return fail(AB200_EINVAL, "ring_depth must be 0 (auto) or a multiple of 4 up to %d", R_MAX_DEPTH);
  g_ring_depth = d;
  return AB200_OK;
}

bool gemv_ring_eligible(int M, int K, int N, int group, bool tiled) {
  if (M != 1 || group != 128 || K % 128 != 0 || N % TILE_N != 0 || K < 128) return false;
  if (!tiled && tensor_map_encoder() == nullptr) return false;
  return true;
}

template <int EPI, int PRO>
static int launch_ring(const CUtensorMap &tm, const RingParams &p, int tiles, int cs, size_t smem, cudaStream_t stream) {
  auto kern = w4a16_gemv_ring_kernel<EPI, PRO, false>;
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * cs, 1, 1);
  cfg.blockDim = dim3(R_THREADS, 1, 1);
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
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm, p, (const RingParams *)nullptr, 0));
  return AB200_OK;
}

template <int PRO>
static int ring_by_epi(const CUtensorMap &tm, const RingParams &p, int tiles, int cs, size_t smem, int epi, cudaStream_t s) {
  if (epi == EPI_STORE) return launch_ring<EPI_STORE, PRO>(tm, p, tiles, cs, smem, s);
  if (epi == EPI_RESIDUAL) return launch_ring<EPI_RESIDUAL, PRO>(tm, p, tiles, cs, smem, s);
  if (epi == EPI_ALLREDUCE) {
    if (PRO == PRO_RMSNORM) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: the fused all-reduce serves the plain and SiLU*up prologues");
    return launch_ring<EPI_ALLREDUCE, PRO == PRO_RMSNORM ? PRO_PLAIN : PRO>(tm, p, tiles, cs, smem, s);
  }
  return launch_ring<EPI_STORE_F32, PRO>(tm, p, tiles, cs, smem, s);
}

struct RingPlan {
  int tiles, cs, depth, nst_max;
  size_t smem;
};

static int ring_plan(int K, int N, RingPlan &pl) {
  const int tiles = N / TILE_N, groups = K / 128;
  int cs = gemv_tuning_cluster();
  if (cs <= 0) {
    // enough CTAs for two per SM, as long as every CTA keeps at least two stages
    const int target = 2 * sm_count();
    cs = 1;
    while (cs < 8 && tiles * cs < target && groups / (cs * 2) >= 2) cs *= 2;
  }
  while (cs > 1 && groups / cs < 1) cs /= 2;
  const int nst_max = (groups + cs - 1) / cs;
  // ring depth: as deep as lets every CTA of the grid be resident at once (a multiple of 4 stages)
  const size_t fixed = (size_t)nst_max * (R_SCALE_ROW_BYTES + 256 + 16) + (size_t)(R_CWARPS + 1) * TILE_N * sizeof(float);
  int depth = g_ring_depth;
  if (depth == 0) {
    int per_sm = (tiles * cs + sm_count() - 1) / sm_count();
    if (per_sm > 4) per_sm = 4;
    const size_t budget = (size_t)225 * 1024 / per_sm - 1024;
    depth = budget > fixed ? (int)((budget - fixed) / R_STAGE_BYTES) & ~3 : 4;
    if (depth > 12) depth = 12;
  }
  if (depth > ((nst_max + 3) & ~3)) depth = (nst_max + 3) & ~3;
  if (depth < 4) depth = 4;
  pl.tiles = tiles;
  pl.cs = cs;
  pl.depth = depth;
  pl.nst_max = nst_max;
  pl.smem = (size_t)depth * R_STAGE_BYTES + fixed;
  if (pl.smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: K slice of %d groups does not fit shared memory", nst_max);
  return AB200_OK;
}

static int ring_params(RingParams &p, const void *x, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int K,
                       int N, bool tiled, int depth) {
  p = RingParams{};
  p.x = x;
  p.norm_w = norm_w;
  p.qw = qw;
  p.scales = reinterpret_cast<const __half *>(scales);
  p.out = out;
  p.status = kernel_error_ptr();
  if (!p.status) return fail(AB200_ECUDA, "w4a16_gemv: status word unavailable");
  p.K = K;
  p.N = N;
  p.groups = K / 128;
  p.depth = depth;
  p.tiled = tiled ? 1 : 0;
  p.pdl_late = pdl_mode() == 2;
  p.eps = eps;
  p.wait_polls = g_ring_wait_polls;
  return AB200_OK;
}

// Receive buffer of comm.cu: uint2 slots[2][world][n_max]; int epoch; int ticket; ...
static void ring_comm(RingParams &p, void *const *bufs, int rank, int world, int n_max) {
  for (int q = 0; q < world; ++q) p.slots[q] = reinterpret_cast<uint2 *>(bufs[q]);
  p.epoch = reinterpret_cast<int *>(reinterpret_cast<char *>(bufs[rank]) + (size_t)2 * world * n_max * sizeof(uint2));
  p.rank = rank;
  p.world = world;
  p.n_max = n_max;
  p.comm_polls = comm_wait_polls();
}

// The caller has checked gemv_ring_eligible.  comm_bufs != nullptr with epi == EPI_ALLREDUCE.
int gemv_ring_dispatch(const void *x, int pro, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int K, int N,
                       int epi, bool tiled, cudaStream_t s, void *const *comm_bufs, int rank, int world, int n_max) {
  RingPlan pl;
  if (int rc = ring_plan(K, N, pl)) return rc;
  RingParams p;
  if (int rc = ring_params(p, x, norm_w, eps, qw, scales, out, K, N, tiled, pl.depth)) return rc;
  if (epi == EPI_ALLREDUCE) ring_comm(p, comm_bufs, rank, world, n_max);
  CUtensorMap tm;
  memset(&tm, 0, sizeof(tm));
  if (!tiled) {
    RingEncodeFn enc = reinterpret_cast<RingEncodeFn>(tensor_map_encoder());
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 8)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    const cuuint32_t box[2] = {TILE_N, R_STAGE_ROWS}, estr[2] = {1, 1};
    const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(qw), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AB200_ECUDA, "w4a16_gemv: cuTensorMapEncodeTiled(qweight) failed with %d", (int)r);
  }
  if (pro == PRO_PLAIN) return ring_by_epi<PRO_PLAIN>(tm, p, pl.tiles, pl.cs, pl.smem, epi, s);
  if (pro == PRO_RMSNORM) return ring_by_epi<PRO_RMSNORM>(tm, p, pl.tiles, pl.cs, pl.smem, epi, s);
  return ring_by_epi<PRO_SILU_MUL>(tm, p, pl.tiles, pl.cs, pl.smem, epi, s);
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_w4a16_gemv_tiled_allreduce(const void *x, int prologue, const int32_t *qweight_tiled, const void *scales_tiled,
                                                float *resid_f32, int K, int N, int group, void *const *bufs_host, int rank, int world,
                                                int n_max, void *stream) {
  clear_error();
  AB200_REQUIRE(x && qweight_tiled && scales_tiled && resid_f32 && bufs_host, "w4a16_gemv_tiled_allreduce: null pointer");
  AB200_REQUIRE(prologue == PRO_PLAIN || prologue == PRO_SILU_MUL, "w4a16_gemv_tiled_allreduce: prologue %d (0 plain or 2 SiLU*up)", prologue);
  AB200_REQUIRE(world >= 1 && world <= R_MAX_WORLD && rank >= 0 && rank < world, "w4a16_gemv_tiled_allreduce: rank %d / world %d", rank, world);
  AB200_REQUIRE(gemv_ring_eligible(1, K, N, group, true), "w4a16_gemv_tiled_allreduce: needs group 128, K %% 128 == 0, N %% 128 == 0 (K=%d N=%d group=%d)", K, N, group);
  AB200_REQUIRE(N <= n_max, "w4a16_gemv_tiled_allreduce: N=%d exceeds the exchange buffer's n_max=%d", N, n_max);
  AB200_REQUIRE(aligned16(x) && aligned16(qweight_tiled) && aligned16(scales_tiled) && aligned16(resid_f32), "w4a16_gemv_tiled_allreduce: pointers must be 16-byte aligned");
  return gemv_ring_dispatch(x, prologue, nullptr, 0.f, qweight_tiled, scales_tiled, resid_f32, K, N, world == 1 ? (int)EPI_RESIDUAL : (int)EPI_ALLREDUCE, true,
                            (cudaStream_t)stream, bufs_host, rank, world, n_max);
}

extern "C" int ab200_w4a16_gemv_tiled_allreduce_emulated(const void *const *x_host, int prologue, const int32_t *const *qweight_tiled_host,
                                                         const void *const *scales_tiled_host, float *const *resid_host, const int *K_host,
                                                         int N, void *const *bufs_host, int world, int n_max, void *emu_scratch_dev,
                                                         void *stream) {
  clear_error();
  AB200_REQUIRE(x_host && qweight_tiled_host && scales_tiled_host && resid_host && K_host && bufs_host && emu_scratch_dev,
                "w4a16_gemv_tiled_allreduce_emulated: null pointer");
  AB200_REQUIRE(prologue == PRO_PLAIN || prologue == PRO_SILU_MUL, "w4a16_gemv_tiled_allreduce_emulated: prologue %d (0 plain or 2 SiLU*up)", prologue);
  AB200_REQUIRE(world >= 2 && world <= R_MAX_WORLD && N <= n_max, "w4a16_gemv_tiled_allreduce_emulated: world %d, N %d, n_max %d", world, N, n_max);
  int k_min = K_host[0], k_max = K_host[0];
  for (int r = 0; r < world; ++r) {
    AB200_REQUIRE(gemv_ring_eligible(1, K_host[r], N, 128, true), "w4a16_gemv_tiled_allreduce_emulated: K=%d N=%d outside the kernel's shapes", K_host[r], N);
    k_min = K_host[r] < k_min ? K_host[r] : k_min;
    k_max = K_host[r] > k_max ? K_host[r] : k_max;
  }
  RingPlan pl, pl_max;
  if (int rc = ring_plan(k_min, N, pl)) return rc;      // the K split every rank can serve
  {
    const int nst_max = (k_max / 128 + pl.cs - 1) / pl.cs;  // shared memory for the longest slice
    pl_max = pl;
    pl_max.smem = (size_t)pl.depth * R_STAGE_BYTES + (size_t)nst_max * (R_SCALE_ROW_BYTES + 256 + 16) + (size_t)(R_CWARPS + 1) * TILE_N * sizeof(float);
    if (pl_max.smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv_tiled_allreduce_emulated: K slice does not fit shared memory");
  }
  RingParams ps[R_MAX_WORLD];
  for (int r = 0; r < world; ++r) {
    if (int rc = ring_params(ps[r], x_host[r], nullptr, 0.f, qweight_tiled_host[r], scales_tiled_host[r], resid_host[r], K_host[r], N, true, pl.depth)) return rc;
    ring_comm(ps[r], bufs_host, r, world, n_max);
  }
  AB200_CUDA(cudaMemcpyAsync(emu_scratch_dev, ps, sizeof(RingParams) * world, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  AB200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));  // `ps` is a stack object
  auto kern = (prologue == PRO_PLAIN) ? w4a16_gemv_ring_kernel<EPI_ALLREDUCE, PRO_PLAIN, true> : w4a16_gemv_ring_kernel<EPI_ALLREDUCE, PRO_SILU_MUL, true>;
  if (pl_max.smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  const int ctas_per_rank = pl.tiles * pl.cs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas_per_rank * world, 1, 1);
  cfg.blockDim = dim3(R_THREADS, 1, 1);
  cfg.dynamicSmemBytes = pl_max.smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;  // the ranks' CTAs wait on one another: all must be resident
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  CUtensorMap tm;
  memset(&tm, 0, sizeof(tm));
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm, ps[0], reinterpret_cast<const RingParams *>(emu_scratch_dev), ctas_per_rank));
  return AB200_OK;
}

extern "C" size_t ab200_w4a16_gemv_emulation_scratch_bytes(void) { return sizeof(RingParams) * R_MAX_WORLD; }

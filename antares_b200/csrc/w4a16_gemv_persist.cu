// W4A16 decode GEMV, persistent balanced variant (fp16 activations/scales, batch 1..16).
//
// One CTA per SM (16 warps), launched once per GEMV.  The matrix is cut into work units of
// 32 columns x one K slice (a few quantisation groups); unit u = slice * tiles + tile, so units
// that are neighbours in the order read neighbouring 128-byte chunks of the same packed rows.
// SM i owns the contiguous unit range [U*i/G, U*(i+1)/G) - every SM streams the same number of
// bytes to within one unit - and its warps pull units from a shared-memory counter.  Inside a
// unit the warp streams 4 packed rows x 128 B per load instruction (lane (g,t): 16-byte chunk g
// of packed row 4s+t), with the next 128 k of weights in registers while the current 128 k are
// unpacked (1 SHF + 4 LOP3 per word, 0x6400 fp16 magic, zero-point by HSUB2/HFMA2) and contracted
// with `mma.sync.m16n8k16` (weights = A operand, x = B operand from shared memory).
//
// K slices of one column tile are summed deterministically without any waiting: each unit stores
// its fp32 partial to scratch, fences, and bumps the tile's counter; whichever warp arrives last
// adds the partials in slice order and runs the epilogue, then re-zeroes the counter.
//
// Prologues (how the CTA builds x in shared memory): plain fp16 x; RMSNorm of an fp32 residual
// row (sum of squares + scale, so the normalised vector never goes through HBM); SiLU(gate) * up.
// Epilogues: fp16 store, fp32 store, fp32 residual += fp16-rounded result.
//
// HBM-bound: algorithmic bytes = K*N/2 + (K/group)*N*2 + M*K*2 + M*N*2 per launch.
#include "common.cuh"
#include "gemv_shared.cuh"

namespace ab200 {

constexpr int P_WARPS = 16;
constexpr int P_THREADS = P_WARPS * 32;
constexpr int P_TILE = 32;          // columns per unit
constexpr int CHUNK_STEPS = 4;      // steps (32 k each) per register chunk = one 128-k block
constexpr int P_XPAD = 32;          // halves; batch rows 64 B apart modulo 128 B -> conflict-free LDS.128
constexpr int P_DEPTH = 4;          // 128-k blocks in flight per warp (2 KiB of weights each)
constexpr int P_SLOT_BYTES = CHUNK_STEPS * 512 + 4 * 256;  // weights [4 steps][32 lanes][16 B] + scales [<=4][32 lanes][8 B]

struct PersistParams {
  const void *x;          // PRO_PLAIN: fp16 [M,K]; PRO_RMSNORM: fp32 [M,K]; PRO_SILU_MUL: fp16 [M,2K] (gate | up)
  const __half *norm_w;   // PRO_RMSNORM: fp16 [K]
  const int32_t *qw;
  const __half *scales;
  void *out;
  float *partial;         // scratch [S][M][N] fp32 (unused when S == 1)
  int *counters;          // scratch [tiles] ints, zero on entry, zero on exit
  int M, K, N, group;
  int tiles, S, units128; // units128 = K/128; S = number of K slices
  int bps;                // 128-k blocks per slice (the last slice may be shorter)
  int ring_offset;        // byte offset of the cp.async rings in dynamic shared memory
  int xs_stride;          // halves between batch rows of x in shared memory
  float eps;
};

// MB = 8 or 16 batch rows; SPG = steps per scale group within a 128-k block (4, 2 or 1).
// Requires K % 128 == 0 and N % 4 == 0.  All index arithmetic in the streaming loop is 32-bit
// pointer bumping: no multiplies, no bounds predicates (out-of-range columns are clamped to the
// last valid chunk and dropped at the store; batch rows beyond M read a zero block).
template <int MB, int SPG, int PRO, int EPI>
__global__ void __launch_bounds__(P_THREADS, 1) w4a16_gemv_persist_kernel(PersistParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float sh_red[P_WARPS];
  __shared__ int sh_next;
  constexpr int NB = MB / 8;
  constexpr int NSC = CHUNK_STEPS / SPG;
  // shared memory: [256 B zero block][x rows]
  __half *xs = reinterpret_cast<__half *>(smem_raw + 256);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int M = p.M, K = p.K, N = p.N;
  const int rowsK = K / 8;
  const int xs_stride = p.xs_stride;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int U = p.tiles * p.S;
  const int u_begin = (int)((long)U * blockIdx.x / gridDim.x), u_end = (int)((long)U * (blockIdx.x + 1) / gridDim.x);
  if (threadIdx.x == 0) sh_next = u_begin + P_WARPS;
  if (threadIdx.x < 16) reinterpret_cast<uint4 *>(smem_raw)[threadIdx.x] = make_uint4(0, 0, 0, 0);

  const int group_blocks = p.group >= 128 ? p.group / 128 : 1;  // 128-k blocks per scale row (SPG == 4)
  const int srows_per_block = p.group >= 128 ? 1 : 128 / p.group;

  // Per-warp ring of P_DEPTH blocks in shared memory, filled with cp.async (16 B per lane per
  // step, L2 only).  Each lane copies exactly what it reads back, so completion is tracked per
  // thread with cp.async groups and the ring needs no barrier.
  unsigned char *ring = smem_raw + p.ring_offset + (size_t)warp * P_DEPTH * P_SLOT_BYTES;
  const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + lane * 16u;

  // Load cursor of this warp: unit (tile, slice), next 128-k block b0 of [.., b_end), bumped pointers.
  struct Cursor {
    int b0, b_end, tile, slice;
    const uint4 *wp;   // packed row b0*16 + t, this thread's 16-byte chunk
    const __half *sp;  // scale row of block b0, this thread's 4 columns
    bool valid;
  };
  struct Desc {  // what the compute side needs to know about a block in flight
    int b0, tile, slice;
    bool valid, ends_unit;
  };
  const int n0_max = N - 4;
  const unsigned w_step = (unsigned)N;                      // uint4 elements between packed rows r and r+4
  const unsigned s_step = (unsigned)N * srows_per_block;    // halves between the scale rows of consecutive blocks
  auto open_unit = [&](int uu) {
    Cursor c;
    c.valid = uu < u_end;
    if (!c.valid) uu = u_begin;  // keep pointers in range
    c.slice = uu / p.tiles;
    c.tile = uu - c.slice * p.tiles;
    c.b0 = c.slice * p.bps;
    c.b_end = (c.b0 + p.bps < p.units128) ? c.b0 + p.bps : p.units128;
    int n0 = c.tile * P_TILE + g * 4;
    if (n0 > n0_max) n0 = n0_max;
    c.wp = reinterpret_cast<const uint4 *>(p.qw + (size_t)(c.b0 * 16 + t) * N + n0);
    c.sp = p.scales + (size_t)((SPG == 4) ? (c.b0 / group_blocks) : (c.b0 * srows_per_block)) * N + n0;
    return c;
  };
  auto issue_block = [&](Cursor &c, int slot) {  // copy block c.b0 into ring slot `slot`, then step the cursor
    const uint32_t dst = ring_u32 + slot * P_SLOT_BYTES;
#pragma unroll
    for (int s = 0; s < CHUNK_STEPS; ++s) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + s * 512), "l"(c.wp) : "memory");
      c.wp += w_step;
    }
    const uint32_t sdst = ring_u32 - lane * 8u + slot * P_SLOT_BYTES + CHUNK_STEPS * 512;
#pragma unroll
    for (int i = 0; i < NSC; ++i)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sdst + i * 256), "l"(c.sp + (size_t)i * N) : "memory");
    if (SPG == 4) {
      if (group_blocks == 1 || (c.b0 + 1) % group_blocks == 0) c.sp += s_step;
    } else {
      c.sp += s_step;
    }
  };
  auto describe = [&](const Cursor &c) {
    Desc d;
    d.b0 = c.b0; d.tile = c.tile; d.slice = c.slice;
    d.valid = c.valid;
    d.ends_unit = c.b0 + 1 >= c.b_end;
    return d;
  };
  auto advance = [&](Cursor &c) {  // to the block after b0 (possibly in a new unit)
    if (!c.valid) return;
    if (c.b0 + 1 < c.b_end) {
      c.b0 += 1;
    } else {
      int nu = 0;
      if (lane == 0) nu = atomicAdd(&sh_next, 1);
      nu = __shfl_sync(0xffffffffu, nu, 0);
      c = open_unit(nu);
    }
  };

  __syncthreads();  // sh_next is set
  Cursor ld = open_unit(u_begin + warp);
  Desc dq[P_DEPTH];
#pragma unroll
  for (int i = 0; i < P_DEPTH; ++i) {  // weights are on their way before x exists
    dq[i] = describe(ld);
    if (ld.valid) issue_block(ld, i);
    asm volatile("cp.async.commit_group;" ::: "memory");
    advance(ld);
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- prologue: build x in shared memory ----------------------------------------------------------
  if (PRO == PRO_PLAIN) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < M * rowsK; i += P_THREADS) {
      const int m = i / rowsK, r = i - m * rowsK;
      *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) =
          permute_row(*reinterpret_cast<const uint4 *>(xg + (size_t)m * K + r * 8));
    }
  } else if (PRO == PRO_SILU_MUL) {
    const __half *xg = reinterpret_cast<const __half *>(p.x);
    for (int i = threadIdx.x; i < M * rowsK; i += P_THREADS) {
      const int m = i / rowsK, r = i - m * rowsK;
      const uint4 gv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + r * 8);
      const uint4 uv = *reinterpret_cast<const uint4 *>(xg + (size_t)m * 2 * K + K + r * 8);
      const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(u2h2(ga[j])), uf = __half22float2(u2h2(ua[j]));
        o[j] = h22u(__floats2half2_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y));
      }
      *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = permute_row(make_uint4(o[0], o[1], o[2], o[3]));
    }
  } else {  // PRO_RMSNORM: one batch row at a time
    const float *xg = reinterpret_cast<const float *>(p.x);
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int r = threadIdx.x; r < rowsK; r += P_THREADS) {
        const float4 a = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8);
        const float4 b = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8 + 4);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) sh_red[warp] = ss;
      __syncthreads();
      float tot = (lane < P_WARPS) ? sh_red[lane] : 0.f;
      tot = warp_sum(tot);
      __syncthreads();
      const float rs = rsqrtf(tot * (1.0f / (float)K) + p.eps);
      for (int r = threadIdx.x; r < rowsK; r += P_THREADS) {
        const float4 a = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8);
        const float4 b = *reinterpret_cast<const float4 *>(xg + (size_t)m * K + r * 8 + 4);
        const uint4 wv = *reinterpret_cast<const uint4 *>(p.norm_w + r * 8);
        const float2 w0 = __half22float2(u2h2(wv.x)), w1 = __half22float2(u2h2(wv.y)), w2 = __half22float2(u2h2(wv.z)),
                     w3 = __half22float2(u2h2(wv.w));
        uint4 o;
        o.x = h22u(__floats2half2_rn(a.x * rs * w0.x, a.y * rs * w0.y));
        o.y = h22u(__floats2half2_rn(a.z * rs * w1.x, a.w * rs * w1.y));
        o.z = h22u(__floats2half2_rn(b.x * rs * w2.x, b.y * rs * w2.y));
        o.w = h22u(__floats2half2_rn(b.z * rs * w3.x, b.w * rs * w3.y));
        *reinterpret_cast<uint4 *>(xs + (size_t)m * xs_stride + r * 8) = permute_row(o);
      }
    }
  }
  __syncthreads();

  // ---- streaming loop ----------------------------------------------------------------------------------
  // Shared-memory byte address of this lane's x operand for block 0 (batch row g [+8]; lanes whose
  // row is beyond M read the zero block and never advance).
  const uint32_t xs_base = (uint32_t)__cvta_generic_to_shared(xs);
  const uint32_t zero_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  uint32_t x_row[NB], x_blk[NB];  // base address of the lane's batch row (+ t*16), bytes per 128-k block (256 or 0)
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = g + nb * 8;
    const bool ok = m < M;
    x_row[nb] = ok ? xs_base + (uint32_t)(m * xs_stride) * 2u + t * 16u : zero_base + t * 16u;
    x_blk[nb] = ok ? 256u : 0u;
  }

  float facc[NB][2][4];
  auto zero_acc = [&]() {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) facc[nb][j][i] = 0.f;
  };
  zero_acc();

  auto compute_block = [&](int slot, int b0) {
    const uint32_t src = ring_u32 + slot * P_SLOT_BYTES;
    float d[NB][2][4];
    uint32_t xa[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) xa[nb] = x_row[nb] + (uint32_t)b0 * x_blk[nb];
#pragma unroll
    for (int s = 0; s < CHUNK_STEPS; ++s) {
      if (s % SPG == 0) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) d[nb][j][i] = 0.f;
      }
      uint4 xb[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) xb[nb] = lds128(xa[nb] + s * 64);
      const uint4 wv = lds128(src + s * 512);
      const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t lo[4], hi[4];
        unpack_pair(wr[2 * j], wr[2 * j + 1], lo, hi);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma16816p(d[nb][j], lo[0], lo[1], lo[2], lo[3], xb[nb].x, xb[nb].y);
          mma16816p(d[nb][j], hi[0], hi[1], hi[2], hi[3], xb[nb].z, xb[nb].w);
        }
      }
      if (s % SPG == SPG - 1) {
        uint2 sv;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(sv.x), "=r"(sv.y) : "r"(src - lane * 8u + CHUNK_STEPS * 512 + (s / SPG) * 256));
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
  };

  // facc[nb][j][i]: column n0 + 2j + (i>>1), batch nb*8 + 2t + (i&1).
  auto epilogue = [&](int m, int n0, float4 v) {
    const size_t o = (size_t)m * N + n0;
    if (EPI == EPI_STORE) {
      uint2 h;
      h.x = h22u(__floats2half2_rn(v.x, v.y));
      h.y = h22u(__floats2half2_rn(v.z, v.w));
      *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.out) + o) = h;
    } else if (EPI == EPI_STORE_F32) {
      *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + o) = v;
    } else {
      float4 r = *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + o);
      r.x += __half2float(__float2half_rn(v.x));
      r.y += __half2float(__float2half_rn(v.y));
      r.z += __half2float(__float2half_rn(v.z));
      r.w += __half2float(__float2half_rn(v.w));
      *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + o) = r;
    }
  };
  auto finish_unit = [&](int tile, int slice) {
    const int n0 = tile * P_TILE + g * 4;
    const bool col_ok = n0 < N;
    // this thread's values for batch row m = nb*8 + 2t + b are columns n0..n0+3
    if (p.S == 1) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int m = nb * 8 + 2 * t + b;
          if (m < M && col_ok) epilogue(m, n0, make_float4(facc[nb][0][b], facc[nb][0][2 + b], facc[nb][1][b], facc[nb][1][2 + b]));
        }
    } else {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int m = nb * 8 + 2 * t + b;
          if (m < M && col_ok)
            *reinterpret_cast<float4 *>(p.partial + ((size_t)slice * M + m) * N + n0) =
                make_float4(facc[nb][0][b], facc[nb][0][2 + b], facc[nb][1][b], facc[nb][1][2 + b]);
        }
      __threadfence();
      __syncwarp();
      int old = 0;
      if (lane == 0) old = atomicAdd(p.counters + tile, 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old == p.S - 1) {  // last slice of this tile to arrive: add all slices in slice order
        __threadfence();
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int m = nb * 8 + 2 * t + b;
            if (m < M && col_ok) {
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int s = 0; s < p.S; ++s) {
                const float4 v = ldcg_f4(p.partial + ((size_t)s * M + m) * N + n0);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
              }
              epilogue(m, n0, acc);
            }
          }
        if (lane == 0) p.counters[tile] = 0;
      }
    }
    zero_acc();
  };

  for (;;) {
    bool done = false;
#pragma unroll
    for (int i = 0; i < P_DEPTH; ++i) {
      if (!dq[i].valid) { done = true; break; }
      asm volatile("cp.async.wait_group %0;" ::"n"(P_DEPTH - 1) : "memory");  // this thread's copies of block dq[i] landed
      compute_block(i, dq[i].b0);
      if (dq[i].ends_unit) finish_unit(dq[i].tile, dq[i].slice);
      dq[i] = describe(ld);
      if (ld.valid) issue_block(ld, i);  // refill the slot just drained (same thread wrote and read it)
      asm volatile("cp.async.commit_group;" ::: "memory");
      advance(ld);
    }
    if (done) break;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- host side -------------------------------------------------------------------------------------

// 128-k blocks per K slice: the largest power of two (>= 2 when possible) that still leaves about one
// unit per warp on every SM.
static int pick_bps(int tiles, int units128, int sms) {
  int bps = 1;
  while (bps * 2 <= units128) bps *= 2;
  while (bps > 2 && (long)tiles * ((units128 + bps - 1) / bps) < (long)sms * P_WARPS) bps /= 2;
  return bps;
}

static size_t persist_x_bytes(int M, int K) { return 256 + (((size_t)M * (K + P_XPAD) * 2 + 127) & ~(size_t)127); }
static size_t persist_smem_bytes(int M, int K) { return persist_x_bytes(M, K) + (size_t)P_WARPS * P_DEPTH * P_SLOT_BYTES; }

size_t gemv_persist_scratch_bytes(int M, int K, int N) {
  const int tiles = (N + P_TILE - 1) / P_TILE;
  const int units128 = K / 128;
  const int bps = pick_bps(tiles, units128 > 0 ? units128 : 1, sm_count());
  const int S = (units128 + bps - 1) / bps;
  return PERSIST_COUNTER_BYTES + (size_t)(S > 1 ? S : 1) * M * N * sizeof(float);
}

bool gemv_persist_fits(int M, int K, int N) {
  return K % 128 == 0 && N >= 4 && persist_smem_bytes(M, K) <= 226 * 1024 &&
         (size_t)((N + P_TILE - 1) / P_TILE) * sizeof(int) <= PERSIST_COUNTER_BYTES;
}

template <int MB, int SPG, int PRO, int EPI>
static int launch_persist(PersistParams p, cudaStream_t stream) {
  auto kern = w4a16_gemv_persist_kernel<MB, SPG, PRO, EPI>;
  p.xs_stride = p.K + P_XPAD;
  p.ring_offset = (int)persist_x_bytes(p.M, p.K);
  const size_t smem = persist_smem_bytes(p.M, p.K);
  if (smem > 226 * 1024) return fail(AB200_EUNSUPPORTED, "w4a16_gemv: x of %d x %d does not fit shared memory", p.M, p.K);
  AB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  int grid = sm_count();
  const int U = p.tiles * p.S;
  if (grid > U) grid = U;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(P_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return AB200_OK;
}

template <int MB, int PRO, int EPI>
static int persist_by_group(const PersistParams &p, cudaStream_t s) {
  if (p.group % 128 == 0) return launch_persist<MB, 4, PRO, EPI>(p, s);
  if (p.group % 64 == 0) return launch_persist<MB, 2, PRO, EPI>(p, s);
  return launch_persist<MB, 1, PRO, EPI>(p, s);
}

template <int PRO, int EPI>
static int persist_by_batch(const PersistParams &p, cudaStream_t s) {
  return (p.M <= 8) ? persist_by_group<8, PRO, EPI>(p, s) : persist_by_group<16, PRO, EPI>(p, s);
}

// scratch: at least gemv_persist_scratch_bytes(M, K, N) bytes, 16-byte aligned; its counter region (the
// first PERSIST_COUNTER_BYTES) must be zero on entry and is zero again on exit.
int gemv_persist_dispatch(const void *x, const __half *norm_w, float eps, const int32_t *qw, const void *scales, void *out, int M,
                          int K, int N, int group, int pro, int epi, void *scratch, cudaStream_t s) {
  PersistParams p{};
  p.x = x;
  p.norm_w = norm_w;
  p.qw = qw;
  p.scales = reinterpret_cast<const __half *>(scales);
  p.out = out;
  p.M = M; p.K = K; p.N = N; p.group = group;
  p.tiles = (N + P_TILE - 1) / P_TILE;
  p.units128 = K / 128;
  p.bps = pick_bps(p.tiles, p.units128, sm_count());
  p.S = (p.units128 + p.bps - 1) / p.bps;
  p.counters = reinterpret_cast<int *>(scratch);
  p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + PERSIST_COUNTER_BYTES);
  p.eps = eps;
#define AB200_P_EPI(PRO)                                                      \
  (epi == EPI_STORE      ? persist_by_batch<PRO, EPI_STORE>(p, s)             \
   : epi == EPI_RESIDUAL ? persist_by_batch<PRO, EPI_RESIDUAL>(p, s)          \
                         : persist_by_batch<PRO, EPI_STORE_F32>(p, s))
  if (pro == PRO_PLAIN) return AB200_P_EPI(PRO_PLAIN);
  if (pro == PRO_RMSNORM) return AB200_P_EPI(PRO_RMSNORM);
  return AB200_P_EPI(PRO_SILU_MUL);
#undef AB200_P_EPI
}

}  // namespace ab200

// ---- entry point that allocates nothing ------------------------------------------------------------
// Scratch for ab200_w4a16_gemv_static: lives in the library image, so every GPU that loads the
// library holds it until the process exits.  Layout as for any other scratch of this kernel:
// [64 KiB tile counters][K-slice partial sums].
namespace {
constexpr size_t STATIC_SCRATCH_BYTES = ab200::PERSIST_COUNTER_BYTES + (size_t)2 * 1024 * 1024;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the
// address is looked up once per device (with that device current) and cached here.
static void *g_static_scratch_ptr[64] = {nullptr};
}  // namespace

extern "C" int ab200_w4a16_gemv_static(const void *x, const int32_t *qweight, const void *scales, void *out, int M, int K, int N,
                                       int group, void *stream) {
  using namespace ab200;
  clear_error();
  AB200_REQUIRE(x && qweight && scales && out, "w4a16_gemv_static: null pointer");
  AB200_REQUIRE(M >= 1 && M <= 16, "w4a16_gemv_static: M=%d outside 1..16", M);
  AB200_REQUIRE(K > 0 && K % 128 == 0, "w4a16_gemv_static: K=%d must be a positive multiple of 128", K);
  AB200_REQUIRE(group > 0 && group % 32 == 0 && K % group == 0, "w4a16_gemv_static: group=%d must be a multiple of 32 dividing K=%d", group, K);
  AB200_REQUIRE(N > 0 && N % 4 == 0, "w4a16_gemv_static: N=%d must be a positive multiple of 4", N);
  AB200_REQUIRE(aligned16(x) && aligned16(qweight) && aligned16(scales) && aligned16(out), "w4a16_gemv_static: pointers must be 16-byte aligned");
  if (!gemv_persist_fits(M, K, N))
    return fail(AB200_EUNSUPPORTED, "w4a16_gemv_static: x of %d x %d does not fit the kernel's shared memory", M, K);
  const size_t need = gemv_persist_scratch_bytes(M, K, N);
  if (need > STATIC_SCRATCH_BYTES)
    return fail(AB200_EINVAL, "w4a16_gemv_static: M=%d K=%d N=%d needs %zu bytes of scratch, the built-in scratch holds %zu", M, K, N, need,
                (size_t)STATIC_SCRATCH_BYTES);
  int dev = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(AB200_EUNSUPPORTED, "w4a16_gemv_static: device index %d out of range", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {  // first call on this device: resolve the symbol's device address
    void *ptr = nullptr;
    AB200_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_static_scratch_ptr[dev] = ptr;
  }
  void *scratch = g_static_scratch_ptr[dev];
  // The array keeps whatever the last call left: the tile counters must start at zero.
  const size_t counter_bytes = (size_t)((N + P_TILE - 1) / P_TILE) * sizeof(int);
  AB200_CUDA(cudaMemsetAsync(scratch, 0, counter_bytes, (cudaStream_t)stream));
  return gemv_persist_dispatch(x, nullptr, 0.f, qweight, scales, out, M, K, N, group, PRO_PLAIN, EPI_STORE, scratch, (cudaStream_t)stream);
}

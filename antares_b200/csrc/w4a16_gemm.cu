// W4A16 prefill GEMM on the 5th-generation tensor cores: out[M,N] = x[M,K] . dequant(qweight, scales)
// with fp16 x / scales / out and fp32 accumulation in tensor memory.
//
// Replaces the exported op of samples/05_llama2_7b_int4.py:135-144 when it is called with a leading
// M axis larger than the decode path handles.  The dequantised weight fed to the tensor cores is
// exactly w = RN_fp16(scale * fp16(q - 8)) (IR statement 2), the products accumulate in fp32.
//
// CTA tile 256 (M) x 256 (N), K step 64, three shared-memory stages, 512 + 96 threads, one CTA per SM.
// The two 128-row halves of the tile have their own fp32 accumulator (2 x 256 TMEM columns) and
// share every dequantised weight tile, which halves the dequantisation work per flop against a
// 128-row tile.  All 512 threads fill a stage:
//   A: the x tile arrives by TMA (`cp.async.bulk.tensor.2d`, one box of 64 k x 128 rows per
//      accumulator half, 128-byte swizzle, completion on the stage's mbarrier): whole 128-byte lines
//      from L2, no thread instructions, and the K-major 128B-swizzled layout the MMA reads natively;
//   B: thread t owns column n0 + t % 256 and four of the stage's eight packed rows: each packed
//      int32 word (8 consecutive k of one column) becomes one 16-byte row of a K-major no-swizzle
//      core matrix (LOP3 + 0x6400 magic, HSUB2/HFMA2 for the zero-point, HMUL2 by the group scale,
//      PRMT back to natural k order), so no transpose is needed and a quarter-warp writes 128
//      contiguous bytes.
// Per stage eight `tcgen05.mma.cta_group::1.kind::f16` (M128 N256 K16, both operands K-major; four K steps
// x two accumulators) are issued and committed to the stage's mbarrier; a stage is refilled once the MMAs
// that read it three iterations ago have completed, so filling overlaps the MMAs of the two stages before.
// Issuing is not free for the issuing thread (descriptors pass through uniform registers, every wait and
// commit is a dependent instruction): with one thread doing everything a k tile cost that thread more
// cycles than the tensor pipe needs for its eight MMAs.  So three single-thread roles live in warps 16-18:
// the MMAs of accumulator 0, the MMAs of accumulator 1 (each commits on its own; the barriers count two
// arrivals), and the TMA copies of x, which run up to four k tiles ahead.  Producers and issuers meet only
// through mbarriers (weights ready, x tile landed, MMAs done), there is no block-wide barrier inside the
// K loop.  The epilogue reads the accumulators with `tcgen05.ld` (row = TMEM lane; the four warps that
// share a lane quarter split the 512 columns), rounds to fp16 and stores.
// Short prompts: an accumulator whose 128 rows all lie beyond M is left out (its issuing thread only keeps
// the barriers in step), and when the problem has fewer tiles than half the SMs the grid's z dimension
// splits K into up to four ranges: every CTA stores its fp32 accumulators as partial sums (laid out so
// that a warp's 32 rows of 16 columns are consecutive), the last CTA of a tile to arrive adds the parts in
// part order - bitwise repeatable - and runs the epilogue.
// Every mbarrier wait is bounded and reports through the status word.
#include <cuda.h>  // CUtensorMap and its enums (types only)

#include "common.cuh"

namespace ab200 {

constexpr int GM_BM = 256, GM_BN = 256, GM_BK = 64;
constexpr int GM_HM = 128;                     // rows per accumulator (one MMA's M)
constexpr int GM_FILL_THREADS = 512;               // 16 warps dequantise weights
constexpr int GM_THREADS = GM_FILL_THREADS + 96;   // + three warps whose lane 0 issues: the MMAs of accumulator 0, of accumulator 1, the TMA copies
constexpr int GM_STAGES = 3;    // stages of dequantised weights
constexpr int GM_ASTAGES = 4;   // stages of the x tile: one more, so that its TMA copy is issued two k tiles ahead
constexpr int GM_AH_BYTES = GM_HM * GM_BK * 2;  // 16 KiB: one 128-row half of the x tile (128 rows x 128 B)
constexpr int GM_A_BYTES = 2 * GM_AH_BYTES;    // 32 KiB
constexpr int GM_B_BYTES = GM_BN * GM_BK * 2;  // 32 KiB
constexpr unsigned GM_WAIT_POLLS = 1u << 22;

struct GemmParams {
  const __half *x;
  const int32_t *qw;
  const __half *scales;
  __half *out;
  int M, K, N, group;
  int *status;
  int parts;           // K ranges per tile: > 1 when there are too few tiles to fill the GPU
  float *partial;      // [tiles][parts][16 column chunks][256 rows][16] fp32: K-split partial accumulators
  unsigned *counters;  // [tiles], zero between launches
};

__device__ __forceinline__ uint32_t gm_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes;
// LBO = bytes between the two 16-byte K chunks of one MMA, SBO = bytes between 8-row groups.
__device__ __forceinline__ uint64_t gm_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  return d;                // base offset 0, layout type 0 (no swizzle)
}

// K-major operand in the 128-byte-swizzled layout TMA writes (rows of 128 B, 8-row atoms of 1024 B):
// stride between atoms 1024 B, leading-dimension field unused (1), layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t gm_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ bool gm_mbar_wait(uint64_t *bar, unsigned parity) {
  const uint32_t addr = gm_smem_u32(bar);
  {  // non-blocking probe first: cheaper than try_wait when the phase completed long ago
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  for (unsigned i = 0; i < GM_WAIT_POLLS; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// SPLIT: the grid's z dimension splits K (few tiles); the unsplit instantiation carries none of that code.
template <bool SPLIT>
__global__ void __launch_bounds__(GM_THREADS) w4a16_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x, GemmParams p) {
  extern __shared__ __align__(1024) unsigned char gm_smem_raw[];
  unsigned char *gm_smem = gm_smem_raw + ((1024u - (gm_smem_u32(gm_smem_raw) & 1023u)) & 1023u);  // swizzle atoms need 1024-B alignment
  __shared__ __align__(8) uint64_t mma_bar[GM_STAGES], b_full_bar[GM_STAGES], full_bar[GM_ASTAGES], a_free_bar[GM_ASTAGES];
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s, last_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.y * GM_BM, n0 = blockIdx.x * GM_BN;
  const int K = p.K, N = p.N, M = p.M;
  // K range of this CTA, in k tiles of 64: [kt0, kt0 + ktiles)
  const int kt0 = SPLIT ? (K / GM_BK) * (int)blockIdx.z / p.parts : 0;
  const int ktiles = SPLIT ? (K / GM_BK) * ((int)blockIdx.z + 1) / p.parts - kt0 : K / GM_BK;

  if (tid == 0) {
    for (int s = 0; s < GM_STAGES; ++s)
    {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" ::"r"(gm_smem_u32(&mma_bar[s])));  // one commit per issuing thread
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gm_smem_u32(&b_full_bar[s])), "r"(GM_FILL_THREADS / 32));
    }
    for (int s = 0; s < GM_ASTAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&full_bar[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" ::"r"(gm_smem_u32(&a_free_bar[s])));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fail_s = 0;
  }
  if (warp == 0) {  // one warp allocates both accumulators: all 512 TMEM columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem_u32(&tmem_base_s)), "r"(2 * GM_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_s;

  // instruction descriptor: D fp32, A/B fp16, both K-major, N = 256, M = 128
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(GM_BN >> 3) << 17) | ((uint32_t)(GM_HM >> 4) << 24);

  // ---- per-thread fill roles ---------------------------------------------------------------------------
  // B: column n0 + tid % 256, packed rows bh*4 .. bh*4+3 of the stage's eight.  A column beyond N reads
  // the last column instead: its accumulator columns are never stored.
  const int bcol = tid & (GM_BN - 1), bh = tid >> 8;
  const int nb = min(n0 + bcol, N - 1);
  const int tiles_per_group = p.group / GM_BK;
  const int32_t *qptr = p.qw + nb + (size_t)(kt0 * 8 + bh * 4) * N;  // the packed words of the next k tile to load
  const __half *sptr = p.scales + nb + (size_t)(kt0 / tiles_per_group) * N;  // its scale
  int group_count = kt0 % tiles_per_group;
  const uint32_t b_off = (uint32_t)((bcol >> 3) * 128 + (bcol & 7) * 16 + bh * 4 * (GM_BN / 8) * 128);  // + j * 4096
  // A: thread 0 asks the TMA unit for the two 64 k x 128 row boxes of k tile kt
  auto issue_a = [&](int kt) {
    const int s = kt % GM_ASTAGES;
    const uint32_t bar = gm_smem_u32(&full_bar[s]);
    const uint32_t dst = gm_smem_u32(gm_smem + s * GM_A_BYTES);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(GM_A_BYTES) : "memory");
#pragma unroll
    for (int hm = 0; hm < 2; ++hm)
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst + hm * GM_AH_BYTES),
                   "l"(reinterpret_cast<uint64_t>(&tm_x)), "r"((kt0 + kt) * GM_BK), "r"(m0 + hm * GM_HM), "r"(bar)
                   : "memory");
  };

  // Three register sets for the packed weights: the global loads of k tile kt+3 are issued while
  // tile kt is being written to shared memory.  Loads are issued in k order, so one running pointer
  // (and a counter for the scale row) serves all three sets.
  struct FillRegs {
    uint32_t b[4];
    __half s;
  };
  auto load_next = [&](FillRegs &r) {  // global -> registers for the next k tile
    const int32_t *p0 = qptr, *p1 = p0 + N, *p2 = p1 + N, *p3 = p2 + N;
    // volatile asm: the loads must be ISSUED here, three tiles ahead of their use, not sunk to it
    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(r.b[0]) : "l"(p0));
    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(r.b[1]) : "l"(p1));
    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(r.b[2]) : "l"(p2));
    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(r.b[3]) : "l"(p3));
    unsigned short sbits;
    asm volatile("ld.global.nc.b16 %0, [%1];" : "=h"(sbits) : "l"(sptr));
    r.s = __ushort_as_half(sbits);
    qptr = p3 + (size_t)5 * N;  // eight packed rows on
    if (++group_count == tiles_per_group) {
      group_count = 0;
      sptr += N;
    }
  };

  bool ok = true;
  // Producer warps (0-15): per k tile wait until the MMAs that read the stage three tiles ago are
  // done, write the dequantised weights, make them visible to the tensor core and arrive (one
  // arrive per warp) on the stage's "weights ready" barrier.  No block-wide barrier in the loop:
  // warps drift apart and hide each other's latencies.  `round` = kt / 3; the stage is the call site's.
  auto fill_step = [&](int stage, int round, bool more, FillRegs &r) {
    unsigned char *sb = gm_smem + GM_ASTAGES * GM_A_BYTES + stage * GM_B_BYTES;
    if (round > 0) {
      if (!gm_mbar_wait(&mma_bar[stage], (round - 1) & 1)) {
        ok = false;
        fail_s = 1;
      }
    }
    {
      constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u, MAGIC = 0x64006400u;
      const __half2 c1032 = u2h2(0x64086408u), c16th = u2h2(0x2C002C00u), cm72 = u2h2(0xD480D480u);
      const __half2 sc2 = __half2half2(r.s);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w = r.b[j], w8 = w >> 8;
        uint4 o;  // (k0,k4)(k1,k5)(k2,k6)(k3,k7), each RN_fp16(scale * (q - 8))
        o.x = h22u(__hmul2(__hsub2(u2h2(lop3<0xEA>(w, LO, MAGIC)), c1032), sc2));
        o.y = h22u(__hmul2(__hfma2(u2h2(lop3<0xEA>(w, HI, MAGIC)), c16th, cm72), sc2));
        o.z = h22u(__hmul2(__hsub2(u2h2(lop3<0xEA>(w8, LO, MAGIC)), c1032), sc2));
        o.w = h22u(__hmul2(__hfma2(u2h2(lop3<0xEA>(w8, HI, MAGIC)), c16th, cm72), sc2));
        uint4 n;  // back to natural k order: (k0,k1)(k2,k3)(k4,k5)(k6,k7)
        n.x = __byte_perm(o.x, o.y, 0x5410);
        n.y = __byte_perm(o.z, o.w, 0x5410);
        n.z = __byte_perm(o.x, o.y, 0x7632);
        n.w = __byte_perm(o.z, o.w, 0x7632);
        *reinterpret_cast<uint4 *>(sb + j * (GM_BN / 8) * 128 + b_off) = n;
      }
    }
    if (more) load_next(r);  // this set's next tile: three MMA periods to arrive
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gm_smem_u32(&b_full_bar[stage])) : "memory");
  };
  // Issuers (lane 0 of warps 16 and 17, one per accumulator): the MMAs of a k tile as soon as its weights
  // and its x tile are in shared memory.  Issuing costs the thread tens of cycles per instruction
  // (descriptors through uniform registers, waits, commits), so the work is split over two threads
  // and the TMA copies have a thread of their own.
  auto issue_mmas = [&](int kt, int hm) {
    const int s = kt % GM_STAGES, sA = kt % GM_ASTAGES;
    if (!gm_mbar_wait(&b_full_bar[s], (kt / GM_STAGES) & 1) || !gm_mbar_wait(&full_bar[sA], (kt / GM_ASTAGES) & 1)) {
      ok = false;
      fail_s = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint64_t da0 = gm_desc_sw128(gm_smem_u32(gm_smem + sA * GM_A_BYTES) + hm * GM_AH_BYTES);
    const uint64_t db0 = gm_desc(gm_smem_u32(gm_smem + GM_ASTAGES * GM_A_BYTES + s * GM_B_BYTES), (GM_BN / 8) * 128, 128);
    const uint32_t acc = tmem_acc + hm * GM_BN;
#pragma unroll
    for (int kb = 0; kb < GM_BK / 16; ++kb) {
      // 16 k further: 32 B into the swizzled x row, two 16-byte chunks of (BN/8)*128 B into the weight tile
      const uint64_t da = da0 + (uint64_t)(kb * 2), db = db0 + (uint64_t)(kb * (2 * (GM_BN / 8) * 128 / 16));
      if (kb == 0) {
        const uint32_t accumulate = kt > 0 ? 1u : 0u;
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(acc),
            "l"(da), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u)
            : "memory");
      } else {
        asm volatile(
            "{\n .reg .pred p;\n setp.eq.u32 p, 0, 0;\n"
            " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%4, %4, %4, %4}, p;\n}\n" ::"r"(acc),
            "l"(da), "l"(db), "r"(IDESC), "r"(0u)
            : "memory");
      }
    }
    // arrive on the barriers when every MMA this thread issued so far has completed
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(gm_smem_u32(&mma_bar[s])) : "memory");
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(gm_smem_u32(&a_free_bar[sA])) : "memory");
  };
  if (warp < GM_FILL_THREADS / 32) {
    FillRegs r0, r1, r2;
    load_next(r0);
    if (ktiles > 1) load_next(r1);
    if (ktiles > 2) load_next(r2);
    for (int kt = 0, round = 0; kt < ktiles; kt += 3, ++round) {
      fill_step(0, round, kt + 3 < ktiles, r0);
      if (kt + 1 < ktiles) fill_step(1, round, kt + 4 < ktiles, r1);
      if (kt + 2 < ktiles) fill_step(2, round, kt + 5 < ktiles, r2);
    }
  } else if (lane == 0) {
    const int role = warp - GM_FILL_THREADS / 32;
    if (role < 2 && m0 + role * GM_HM >= M) {
      // this accumulator's rows lie beyond M (a prompt of at most 128 rows): nothing to multiply; arrive in
      // step with the other issuing thread so that the stage barriers still count two arrivals per use
      for (int kt = 0; kt < ktiles; ++kt) {
        const int s = kt % GM_STAGES, sA = kt % GM_ASTAGES;
        if (!gm_mbar_wait(&b_full_bar[s], (kt / GM_STAGES) & 1) || !gm_mbar_wait(&full_bar[sA], (kt / GM_ASTAGES) & 1)) fail_s = 1;
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gm_smem_u32(&mma_bar[s])) : "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gm_smem_u32(&a_free_bar[sA])) : "memory");
      }
    } else if (role < 2) {
      for (int kt = 0; kt < ktiles; ++kt) issue_mmas(kt, role);
    } else {
      // x ring: a stage is refilled as soon as both accumulators' MMAs of four k tiles ago are complete
      for (int kt = 0; kt < ktiles; ++kt) {
        if (kt >= GM_ASTAGES && !gm_mbar_wait(&a_free_bar[kt % GM_ASTAGES], ((kt / GM_ASTAGES) - 1) & 1)) {
          ok = false;
          fail_s = 1;
        }
        issue_a(kt);
      }
    }
  }
  // ---- drain: the last commit covers every MMA -----------------------------------------------------
  {
    const int last = ktiles - 1, s = last % GM_STAGES;
    if (!gm_mbar_wait(&mma_bar[s], (last / GM_STAGES) & 1)) {
      ok = false;
      fail_s = 1;
    }
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  if (fail_s && tid == 0) atomicExch(p.status, 200);

  // ---- epilogue: TMEM -> registers -> fp16 -> shared memory -> global.  A warp reads the TMEM lanes of its
  // quarter (warp % 4); the four warps of a quarter take 128 of the 512 columns each: columns 0-255 are the
  // accumulator of tile rows 0-127, columns 256-511 that of rows 128-255.  A thread holds one row, so storing
  // from registers would scatter 16-byte pieces over 32 rows per instruction; instead the warp parks its
  // 32 x 128 sub-tile in the (now idle) stage memory and writes it back out row by row, 256 contiguous bytes
  // per half-warp.
  // With a K split (few tiles, p.parts > 1) every CTA first stores its fp32 accumulators as partial sums; the
  // last CTA of a tile to arrive adds the parts in part order (bitwise repeatable) and runs the epilogue.
  if (warp < GM_FILL_THREADS / 32) {
    constexpr int ROWB = 128 * 2 + 16;  // bytes per parked row: the pad spreads the lanes' 16-byte stores over the banks
    const int q = warp & 3, cg = warp >> 2;
    const int hm = cg >> 1, c_begin = (cg & 1) * 128;
    unsigned char *park = gm_smem + (size_t)warp * (32 * ROWB);
    const bool rows_live = !fail_s && m0 + hm * GM_HM + q * 32 < M;  // a warp whose 32 rows all lie beyond M has nothing to store
    const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(hm * GM_BN);
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    // partial sums: [tile][part][16-column chunk][256 rows][16] fp32: a warp's 32 rows of one chunk are 2 KiB of consecutive addresses
    float *mine = SPLIT ? p.partial + ((size_t)tile_id * p.parts + blockIdx.z) * (GM_BM * GM_BN) + (size_t)(hm * GM_HM + q * 32 + lane) * 16 : nullptr;
    bool finish = true;
    if (SPLIT) {
      if (rows_live) {
#pragma unroll 2
        for (int c = 0; c < 128; c += 16) {
          uint32_t r[16];
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr + c_begin + c));
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          float4 *dst = reinterpret_cast<float4 *>(mine + (size_t)((c_begin + c) / 16) * (GM_BM * 16));
#pragma unroll
          for (int j = 0; j < 4; ++j)
            __stcg(dst + j, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(GM_FILL_THREADS) : "memory");
      if (tid == 0) {
        const unsigned old = atomicAdd(p.counters + tile_id, 1u);
        const int last = old == (unsigned)(p.parts - 1);
        if (last) p.counters[tile_id] = 0;  // ready for the next launch
        last_s = last;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(GM_FILL_THREADS) : "memory");
      finish = last_s != 0;
      if (finish) __threadfence();
    }
    if (finish && rows_live) {
      const float *all = SPLIT ? p.partial + (size_t)tile_id * p.parts * (GM_BM * GM_BN) + (size_t)(hm * GM_HM + q * 32 + lane) * 16 : nullptr;
#pragma unroll 2
      for (int c = 0; c < 128; c += 16) {
        float v[16];
        if (SPLIT) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          for (int pt0 = 0; pt0 < p.parts; pt0 += 4) {  // four parts' loads in flight together, added in part order
            float4 a[4][4];
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
              const float4 *src = reinterpret_cast<const float4 *>(all + (size_t)(pt0 + pp) * (GM_BM * GM_BN) + (size_t)((c_begin + c) / 16) * (GM_BM * 16));
#pragma unroll
              for (int j = 0; j < 4; ++j) a[pp][j] = pt0 + pp < p.parts ? __ldcg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int pp = 0; pp < 4; ++pp)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                v[4 * j] += a[pp][j].x;
                v[4 * j + 1] += a[pp][j].y;
                v[4 * j + 2] += a[pp][j].z;
                v[4 * j + 3] += a[pp][j].w;
              }
          }
        } else {
          uint32_t r[16];
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr + c_begin + c));
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
        uint4 h0, h1;
        h0.x = h22u(__floats2half2_rn(v[0], v[1]));
        h0.y = h22u(__floats2half2_rn(v[2], v[3]));
        h0.z = h22u(__floats2half2_rn(v[4], v[5]));
        h0.w = h22u(__floats2half2_rn(v[6], v[7]));
        h1.x = h22u(__floats2half2_rn(v[8], v[9]));
        h1.y = h22u(__floats2half2_rn(v[10], v[11]));
        h1.z = h22u(__floats2half2_rn(v[12], v[13]));
        h1.w = h22u(__floats2half2_rn(v[14], v[15]));
        *reinterpret_cast<uint4 *>(park + lane * ROWB + c * 2) = h0;
        *reinterpret_cast<uint4 *>(park + lane * ROWB + c * 2 + 16) = h1;
      }
      __syncwarp();
      const int piece = lane & 15;                       // 16-byte piece (8 columns) of a parked row
      const int col = n0 + c_begin + piece * 8;
      if (col < N) {                                     // N is a multiple of 8: a piece is inside or outside as a whole
#pragma unroll 4
        for (int rr = 0; rr < 32; rr += 2) {
          const int rl = rr + (lane >> 4);
          const int row = m0 + hm * GM_HM + q * 32 + rl;
          const uint4 v = *reinterpret_cast<const uint4 *>(park + rl * ROWB + piece * 16);
          if (row < M) *reinterpret_cast<uint4 *>(p.out + (size_t)row * N + col) = v;
        }
      }
    }
  }
  (void)ok;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(2 * GM_BN) : "memory");
}

// Library-owned scratch for K-split launches: [counters, zero between launches][partial sums]; at most one
// 256 x 256 fp32 tile per SM (37 MiB on 148 SMs).
constexpr size_t GEMM_COUNTER_BYTES = 1024;
static int gemm_scratch(size_t bytes, void **out) { return library_buffer(LIB_BUF_GEMM, bytes, 0, GEMM_COUNTER_BYTES, out); }

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_w4a16_gemm(const void *x, const int32_t *qweight, const void *scales, void *out, int M, int K, int N,
                                int group, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(x && qweight && scales && out, "w4a16_gemm: null pointer");
  if (dtype != AB200_F16) return fail(AB200_EUNSUPPORTED, "w4a16_gemm: the tensor-core path is built for float16 (dtype %d given)", dtype);
  AB200_REQUIRE(M > 0 && N > 0 && N % 8 == 0, "w4a16_gemm: M=%d must be positive, N=%d a positive multiple of 8", M, N);
  AB200_REQUIRE(K > 0 && K % GM_BK == 0, "w4a16_gemm: K=%d must be a positive multiple of %d", K, GM_BK);
  AB200_REQUIRE(group >= GM_BK && group % GM_BK == 0 && K % group == 0, "w4a16_gemm: group=%d must be a multiple of %d dividing K", group, GM_BK);
  AB200_REQUIRE(aligned16(x) && aligned16(qweight) && aligned16(scales) && aligned16(out), "w4a16_gemm: pointers must be 16-byte aligned");
  int *status = kernel_error_ptr();
  AB200_REQUIRE(status != nullptr, "w4a16_gemm: cannot resolve the status word");
  // Few tiles (a short prompt): split K over the idle SMs, at most 4 ranges (the last CTA of a tile adds all
  // parts, one batch of loads per 16 columns) of at least 8 k tiles each
  const int tiles = ((N + GM_BN - 1) / GM_BN) * ((M + GM_BM - 1) / GM_BM), G = sm_count();
  int parts = G / tiles;
  if (parts > 4) parts = 4;
  if (parts > (K / GM_BK) / 8) parts = (K / GM_BK) / 8;
  if (parts < 1) parts = 1;
  void *scratch = nullptr;
  if (parts > 1) {
    if (int rc = gemm_scratch(GEMM_COUNTER_BYTES + (size_t)tiles * parts * GM_BM * GM_BN * sizeof(float), &scratch)) return rc;
  }
  GemmParams p{(const __half *)x, qweight, (const __half *)scales, (__half *)out, M, K, N, group, status, parts,
               scratch ? reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(scratch) + GEMM_COUNTER_BYTES) : nullptr,
               reinterpret_cast<unsigned *>(scratch)};
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);
  EncodeFn enc = reinterpret_cast<EncodeFn>(tensor_map_encoder());
  if (!enc) return fail(AB200_EUNSUPPORTED, "w4a16_gemm: this driver has no cuTensorMapEncodeTiled");
  CUtensorMap tm_x;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {GM_BK, GM_HM}, estr[2] = {1, 1};
    const CUresult r = enc(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AB200_ECUDA, "w4a16_gemm: cuTensorMapEncodeTiled(x) failed with %d", (int)r);
  }
  const size_t smem = (size_t)GM_ASTAGES * GM_A_BYTES + (size_t)GM_STAGES * GM_B_BYTES + 1024;
  AB200_CUDA(cudaFuncSetAttribute(w4a16_gemm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  AB200_CUDA(cudaFuncSetAttribute(w4a16_gemm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const dim3 grid((N + GM_BN - 1) / GM_BN, (M + GM_BM - 1) / GM_BM, parts);
  if (parts > 1) w4a16_gemm_tcgen05_kernel<true><<<grid, GM_THREADS, smem, (cudaStream_t)stream>>>(tm_x, p);
  else w4a16_gemm_tcgen05_kernel<false><<<grid, GM_THREADS, smem, (cudaStream_t)stream>>>(tm_x, p);
  AB200_CHECK_LAUNCH("w4a16_gemm");
  return AB200_OK;
}

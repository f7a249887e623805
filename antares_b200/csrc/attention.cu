// Single-query (decode) attention over an fp16 KV cache, and the dense fp16 classifier GEMV.
// Both are HBM-bound streams: 16-byte loads, fp32 math, warp-shuffle reductions.
#include <math_constants.h>

#include <cooperative_groups.h>

#include "common.cuh"

namespace ab200 {

constexpr int ATT_THREADS = 256;
constexpr int ATT_D = 128;

// 8 consecutive elements as fp32, from fp16 or fp32 storage (streaming loads)
template <typename T>
__device__ __forceinline__ void ld8(const T *p, float (&f)[8]);
__device__ __forceinline__ void h8_to_f8(const uint4 v, float (&f)[8]);
template <>
__device__ __forceinline__ void ld8<__half>(const __half *p, float (&f)[8]) { h8_to_f8(ldg_stream_v4(p), f); }
template <>
__device__ __forceinline__ void ld8<float>(const float *p, float (&f)[8]) {
  const uint4 a = ldg_stream_v4(p), b = ldg_stream_v4(p + 4);
  f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
  f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
}
__device__ __forceinline__ void h8_to_f8(const uint4 v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(u2h2(u[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// One CTA per head.  Replaces autort.ops.attention_f32 (call site
// samples/05_llama2_7b_int4.py:161-165): p = softmax_s(scale * q.K_s), out = sum_s p_s V_s.
// Phase 1: a half-warp per cache row computes the score (16 lanes x 8 dims).
// Phase 2: block-wide max / sum of exp.  Phase 3: 16 row-groups x 16 dim-chunks accumulate P.V.
template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) attention_decode_kernel(const T *__restrict__ q, const T *__restrict__ kc,
                                                                      const T *__restrict__ vc, T *__restrict__ out,
                                                                      const int32_t *__restrict__ seq_len_dev, int seq_len_add,
                                                                      int max_seq, long kv_stride, float scale, KvPages pages) {
  extern __shared__ __align__(16) float att_smem[];
  float *p = att_smem;                // [max_seq]
  float *red = att_smem + max_seq;    // [16][128]
  __shared__ float sh[32];
  const int h = blockIdx.x;
  // blockIdx.y = query row of a causal prefill: row r sees r more cache rows than row 0
  int S = *seq_len_dev + seq_len_add + (int)blockIdx.y;
  S = S < 0 ? 0 : (S > max_seq ? max_seq : S);
  q += (size_t)blockIdx.y * gridDim.x * ATT_D;
  out += (size_t)blockIdx.y * gridDim.x * ATT_D;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 15, hw = lane >> 4;

  float qf[8];
  ld8<T>(q + (size_t)h * ATT_D + sub * 8, qf);
  const T *kh = kc + (size_t)h * ATT_D + sub * 8;
  float mx = -CUDART_INF_F;
  for (int s0 = warp * 2; s0 < S; s0 += 2 * (ATT_THREADS / 32)) {
    const int s = s0 + hw;
    float dot = 0.f;
    if (s < S) {
      float kf[8];
      ld8<T>(kh + kv_row(pages, s) * kv_stride, kf);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot = fmaf(qf[j], kf[j], dot);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (s < S) {
      dot *= scale;
      if (sub == 0) p[s] = dot;
      mx = fmaxf(mx, dot);
    }
  }
  mx = warp_max(mx);
  if (lane == 0) sh[warp] = mx;
  __syncthreads();
  mx = (lane < ATT_THREADS / 32) ? sh[lane] : -CUDART_INF_F;
  mx = warp_max(mx);
  __syncthreads();

  float sum = 0.f;
  for (int s = threadIdx.x; s < S; s += ATT_THREADS) {
    const float e = expf(p[s] - mx);
    p[s] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) sh[warp] = sum;
  __syncthreads();
  sum = (lane < ATT_THREADS / 32) ? sh[lane] : 0.f;
  sum = warp_sum(sum);

  const int dchunk = threadIdx.x & 15, sgroup = threadIdx.x >> 4;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const T *vh = vc + (size_t)h * ATT_D + dchunk * 8;
  for (int s = sgroup; s < S; s += 16) {
    float vf[8];
    ld8<T>(vh + kv_row(pages, s) * kv_stride, vf);
    const float ps = p[s];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = fmaf(ps, vf[j], acc[j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[sgroup * ATT_D + dchunk * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < ATT_D) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 16; ++g) t += red[g * ATT_D + threadIdx.x];
    out[(size_t)h * ATT_D + threadIdx.x] = (T)(S > 0 ? t / sum : 0.f);
  }
}

// Decode-step attention with RoPE and the KV-cache update fused in (replaces the rotary_f32 x2 +
// attention_f32 chain and the cache aliasing of samples/05_llama2_7b_int4.py:151-165).
// Grid = heads x SPLITS; the SPLITS CTAs of one head form a cluster, each takes the cache rows
// s = split, split + SPLITS, ... and they merge their partial softmax (max, sum, weighted V) through
// distributed shared memory.  Every CTA rotates q and the new k of its head itself (128 values);
// the CTA that owns row `pos` writes the rotated k and v into the cache and uses its own copy, so
// nothing is read back from global memory inside the kernel.
// Latency: the position counter and up to 64 cache rows per CTA are fetched into registers before
// griddepcontrol.wait, i.e. while the projection that produces q/k/v is still finishing.  That is
// why the position counter and the cache rows below it must not be written by the kernel that
// immediately precedes this one in the stream (in a decode step they date from earlier steps).
struct AttnFusedParams {
  const __half *vqk;      // [3 * H * D]: V | Q | K of the current token
  const float *inv_freq;  // [D/2 or D]
  const int32_t *pos_dev;
  __half *kc, *vc;        // [max_seq, kv_stride]
  __half *out;            // [H * D]
  int H, max_seq;
  long kv_stride;
  float scale;
  KvPages pages;
};

constexpr int ATT_PF = 4;  // cache rows per thread fetched before the current token's q/k/v exist

__global__ void __launch_bounds__(ATT_THREADS) attention_fused_kernel(AttnFusedParams p) {
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) float att_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int splits = (int)cluster.num_blocks(), split = (int)cluster.block_rank();
  const int h = blockIdx.x / splits;
  float *red = att_smem;                     // [16][128] weighted V per half-warp
  float *inbox = red + 16 * ATT_D;           // [splits][128/splits] weighted V, then [splits] max, [splits] sum
  __shared__ __align__(16) __half q_s[ATT_D], k_s[ATT_D], v_s[ATT_D];
  __shared__ float hw_m[16], hw_l[16];
  const int chunk = threadIdx.x & 15, sgroup = threadIdx.x >> 4;  // 16-byte chunk of a row; row group (16 rows per pass)

  pdl_launch_dependents();
  // Everything up to the wait reads only what earlier steps left behind (the position counter and
  // cache rows below it), so it overlaps the tail of the projection kernel that produces q/k/v.
  const int pos = *p.pos_dev;
  if (pos < 0 || pos >= p.max_seq) {  // out-of-range step: leave cache and output untouched (all CTAs agree)
    return;
  }
  if (splits > 1) cluster_arrive_started();
  const int S = pos + 1;
  const int HD = p.H * ATT_D;
  const int n_local = (S - split + splits - 1) / splits;  // rows split, split+splits, ... < S
  const __half *kh = p.kc + (size_t)h * ATT_D + chunk * 8;
  const __half *vh = p.vc + (size_t)h * ATT_D + chunk * 8;
  uint4 kreg[ATT_PF], vreg[ATT_PF];
#pragma unroll
  for (int j = 0; j < ATT_PF; ++j) {
    const int i = sgroup + 16 * j;
    const int s = split + i * splits;
    kreg[j] = vreg[j] = make_uint4(0, 0, 0, 0);
    if (i < n_local && s != pos) {
      const size_t row = kv_row(p.pages, s);  // the page table, like the rows, dates from earlier steps
      kreg[j] = ldg_stream_v4(kh + row * p.kv_stride);
      vreg[j] = ldg_stream_v4(vh + row * p.kv_stride);
    }
  }
  float sn = 0.f, cs = 1.f;
  if (threadIdx.x < ATT_D / 2) sincosf((float)pos * p.inv_freq[threadIdx.x], &sn, &cs);
  pdl_wait();

  // rotate q and k of this head (rotate-half), keep v
  if (threadIdx.x < ATT_D / 2) {
    const int j = threadIdx.x;
    const __half *q = p.vqk + HD + (size_t)h * ATT_D, *k = p.vqk + 2 * HD + (size_t)h * ATT_D;
    const float qa = __half2float(q[j]), qb = __half2float(q[j + ATT_D / 2]);
    const float ka = __half2float(k[j]), kb = __half2float(k[j + ATT_D / 2]);
    q_s[j] = __float2half_rn(qa * cs - qb * sn);
    q_s[j + ATT_D / 2] = __float2half_rn(qb * cs + qa * sn);
    k_s[j] = __float2half_rn(ka * cs - kb * sn);
    k_s[j + ATT_D / 2] = __float2half_rn(kb * cs + ka * sn);
  } else if (threadIdx.x < ATT_D / 2 + ATT_D / 8) {
    const int i = threadIdx.x - ATT_D / 2;
    reinterpret_cast<uint4 *>(v_s)[i] = reinterpret_cast<const uint4 *>(p.vqk + (size_t)h * ATT_D)[i];
  }
  __syncthreads();
  const bool own_new = (pos % splits) == split;
  if (own_new && threadIdx.x < ATT_D / 8) {
    const size_t row = kv_row(p.pages, pos);
    reinterpret_cast<uint4 *>(p.kc + row * p.kv_stride + (size_t)h * ATT_D)[threadIdx.x] = reinterpret_cast<const uint4 *>(k_s)[threadIdx.x];
    reinterpret_cast<uint4 *>(p.vc + row * p.kv_stride + (size_t)h * ATT_D)[threadIdx.x] = reinterpret_cast<const uint4 *>(v_s)[threadIdx.x];
  }

  // Each half-warp (16 lanes x 8 dims) runs an online softmax over its rows i = sgroup + 16 * pass:
  // running max, running sum and the running weighted V, so scores never go through shared memory.
  float qf[8];
  h8_to_f8(reinterpret_cast<const uint4 *>(q_s)[chunk], qf);
  float m_run = -CUDART_INF_F, l_run = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  auto row_step = [&](bool live, uint4 kv, uint4 vv) {  // called by whole warps; `live` is per half-warp
    float dot = 0.f;
    float kf[8];
    h8_to_f8(kv, kf);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot = fmaf(qf[j], kf[j], dot);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (live) {
      dot *= p.scale;
      const float m_new = fmaxf(m_run, dot);
      const float c = __expf(m_run - m_new), w = __expf(dot - m_new);  // first row: c = exp(-inf) = 0
      float vf[8];
      h8_to_f8(vv, vf);
      l_run = fmaf(l_run, c, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(acc[j], c, w * vf[j]);
      m_run = m_new;
    }
  };
#pragma unroll
  for (int j = 0; j < ATT_PF; ++j) {
    if (16 * j < n_local) {  // uniform over the CTA
      const int i = sgroup + 16 * j;
      const int s = split + i * splits;
      const bool cur = (s == pos);
      row_step(i < n_local, cur ? reinterpret_cast<const uint4 *>(k_s)[chunk] : kreg[j], cur ? reinterpret_cast<const uint4 *>(v_s)[chunk] : vreg[j]);
    }
  }
  for (int i0 = 16 * ATT_PF; i0 < n_local; i0 += 16) {
    const int i = i0 + sgroup;
    const int s = split + i * splits;
    const bool live = i < n_local, cur = (s == pos);
    uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
    if (live) {
      const size_t row = cur ? 0 : kv_row(p.pages, s);
      kv = cur ? reinterpret_cast<const uint4 *>(k_s)[chunk] : ldg_stream_v4(kh + row * p.kv_stride);
      vv = cur ? reinterpret_cast<const uint4 *>(v_s)[chunk] : ldg_stream_v4(vh + row * p.kv_stride);
    }
    row_step(live, kv, vv);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[sgroup * ATT_D + chunk * 8 + j] = acc[j];
  if (chunk == 0) {
    hw_m[sgroup] = m_run;
    hw_l[sgroup] = l_run;
  }
  __syncthreads();
  // merge the 16 half-warp partials per dim, then across the head's CTAs, push model: CTA r stores its
  // un-normalised output slice, max and sum into the inbox of the CTA that finalises those dims; one
  // cluster barrier; local merge.
  const int dims_per = ATT_D / splits;
  if (splits > 1) cluster_wait_started();  // every CTA of the head is running: its inbox may be written
  if (threadIdx.x < ATT_D + splits) {
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int gI = 0; gI < 16; ++gI) mx = fmaxf(mx, hw_m[gI]);
    float l = 0.f, t = 0.f;
    const int d = threadIdx.x < ATT_D ? threadIdx.x : 0;
#pragma unroll
    for (int gI = 0; gI < 16; ++gI) {
      const float mg = hw_m[gI];
      const float w = (mg == -CUDART_INF_F) ? 0.f : __expf(mg - mx);  // a half-warp without rows weighs nothing
      l = fmaf(hw_l[gI], w, l);
      t = fmaf(red[gI * ATT_D + d], w, t);
    }
    if (threadIdx.x < ATT_D) {
      const int owner = threadIdx.x / dims_per, dd = threadIdx.x - owner * dims_per;
      float *dst = (splits > 1) ? cluster.map_shared_rank(inbox, owner) : inbox;
      dst[split * dims_per + dd] = t;
    } else {
      const int owner = threadIdx.x - ATT_D;
      float *dst = (splits > 1) ? cluster.map_shared_rank(inbox, owner) : inbox;
      dst[ATT_D + split] = mx;
      dst[ATT_D + splits + split] = l;
    }
  }
  if (splits > 1) cluster.sync(); else __syncthreads();
  if (threadIdx.x < dims_per) {
    const int d = split * dims_per + threadIdx.x;
    float gm = -CUDART_INF_F;
    for (int r = 0; r < splits; ++r) gm = fmaxf(gm, inbox[ATT_D + r]);
    float l = 0.f, o = 0.f;
    for (int r = 0; r < splits; ++r) {
      const float mr = inbox[ATT_D + r];
      const float w = (mr == -CUDART_INF_F) ? 0.f : __expf(mr - gm);  // a CTA without rows weighs nothing
      l += inbox[ATT_D + splits + r] * w;
      o += inbox[r * dims_per + threadIdx.x] * w;
    }
    p.out[(size_t)h * ATT_D + d] = __float2half_rn(o / l);
  }
}

// logits[n] = W[n, :] . x, W fp16 [N, K] row-major (the classifier matmul,
// samples/05_llama2_7b_int4.py:176).  A warp owns two rows at a time; lanes stride over 16-byte
// chunks of K; x comes through L1.
constexpr int DG_THREADS = 256;
__global__ void __launch_bounds__(DG_THREADS) dense_gemv_kernel(const __half *__restrict__ x, const __half *__restrict__ w,
                                                               float *__restrict__ out, int K, int N) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * (DG_THREADS / 32) + (threadIdx.x >> 5);
  const int n0 = warp_global * 2;
  if (n0 >= N) return;
  const bool two = (n0 + 1) < N;
  const __half *w0 = w + (size_t)n0 * K, *w1 = w + (size_t)(two ? n0 + 1 : n0) * K;
  float a0 = 0.f, a1 = 0.f;
  const int nvec = K / 8;
#pragma unroll 4
  for (int i = lane; i < nvec; i += 32) {
    const uint4 v0 = ldg_stream_v4(w0 + (size_t)i * 8), v1 = ldg_stream_v4(w1 + (size_t)i * 8);
    const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x) + i);
    float xf[8], f0[8], f1[8];
    h8_to_f8(xv, xf);
    h8_to_f8(v0, f0);
    h8_to_f8(v1, f1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a0 = fmaf(xf[j], f0[j], a0);
      a1 = fmaf(xf[j], f1[j], a1);
    }
  }
  a0 = warp_sum(a0);
  a1 = warp_sum(a1);
  if (lane == 0) {
    out[n0] = a0;
    if (two) out[n0 + 1] = a1;
  }
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_attention_decode(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16, void *out_f16,
                                      const int32_t *seq_len_dev, int seq_len_add, int max_seq, int H, int D, long kv_stride,
                                      float scale, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(q_f16 && k_cache_f16 && v_cache_f16 && out_f16 && seq_len_dev, "attention_decode: null pointer");
  AB200_REQUIRE(D == ATT_D, "attention_decode: head size %d is not the built size %d", D, ATT_D);
  AB200_REQUIRE(H > 0 && max_seq > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0, "attention_decode: bad shape H=%d max_seq=%d kv_stride=%ld", H, max_seq, kv_stride);
  AB200_REQUIRE(aligned16(q_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16) && aligned16(out_f16),
                "attention_decode: pointers must be 16-byte aligned");
  const size_t smem = ((size_t)max_seq + 16 * ATT_D) * sizeof(float);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "attention_decode: max_seq=%d exceeds the shared-memory score buffer", max_seq);
  if (dtype == AB200_F16) {
    if (smem > 48 * 1024)
      AB200_CUDA(cudaFuncSetAttribute(attention_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attention_decode_kernel<__half><<<H, ATT_THREADS, smem, (cudaStream_t)stream>>>((const __half *)q_f16, (const __half *)k_cache_f16,
                                                                                   (const __half *)v_cache_f16, (__half *)out_f16, seq_len_dev,
                                                                                   seq_len_add, max_seq, kv_stride, scale, KvPages{nullptr, 0});
  } else if (dtype == AB200_F32) {
    if (smem > 48 * 1024)
      AB200_CUDA(cudaFuncSetAttribute(attention_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attention_decode_kernel<float><<<H, ATT_THREADS, smem, (cudaStream_t)stream>>>((const float *)q_f16, (const float *)k_cache_f16,
                                                                                  (const float *)v_cache_f16, (float *)out_f16, seq_len_dev,
                                                                                  seq_len_add, max_seq, kv_stride, scale, KvPages{nullptr, 0});
  } else {
    return fail(AB200_EINVAL, "attention_decode: unknown dtype %d", dtype);
  }
  AB200_CHECK_LAUNCH("attention_decode");
  return AB200_OK;
}

extern "C" int ab200_dense_gemv(const void *x_f16, const void *w_f16, float *logits_f32, int K, int N, void *stream) {
  clear_error();
  AB200_REQUIRE(x_f16 && w_f16 && logits_f32, "dense_gemv: null pointer");
  AB200_REQUIRE(K > 0 && K % 8 == 0 && N > 0, "dense_gemv: K=%d must be a positive multiple of 8, N=%d positive", K, N);
  AB200_REQUIRE(aligned16(x_f16) && aligned16(w_f16), "dense_gemv: pointers must be 16-byte aligned");
  const int rows_per_block = (DG_THREADS / 32) * 2;
  dense_gemv_kernel<<<(N + rows_per_block - 1) / rows_per_block, DG_THREADS, 0, (cudaStream_t)stream>>>(
      (const __half *)x_f16, (const __half *)w_f16, logits_f32, K, N);
  AB200_CHECK_LAUNCH("dense_gemv");
  return AB200_OK;
}

// page_rows: 0 = contiguous cache, else a power of two (rows per page) with page_table[(max_seq + page_rows - 1) / page_rows]
static int page_shift_of(int page_rows) {
  int shift = 0;
  while ((1 << shift) < page_rows) ++shift;
  return (page_rows > 0 && (1 << shift) == page_rows) ? shift : -1;
}

static int attention_fused_impl(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev, void *k_cache_f16,
                                void *v_cache_f16, void *out_f16, int H, int D, long kv_stride, int max_seq, float scale,
                                const int32_t *page_table, int page_rows, void *stream) {
  clear_error();
  AB200_REQUIRE(page_table == nullptr || page_shift_of(page_rows) >= 0, "attention_fused: page_rows=%d must be a power of two", page_rows);
  AB200_REQUIRE(vqk_f16 && inv_freq && pos_dev && k_cache_f16 && v_cache_f16 && out_f16, "attention_fused: null pointer");
  AB200_REQUIRE(D == ATT_D, "attention_fused: head size %d is not the built size %d", D, ATT_D);
  AB200_REQUIRE(H > 0 && max_seq > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0, "attention_fused: bad shape H=%d max_seq=%d kv_stride=%ld", H, max_seq, kv_stride);
  AB200_REQUIRE(aligned16(vqk_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16) && aligned16(out_f16),
                "attention_fused: pointers must be 16-byte aligned");
  int splits = 1;
  while (splits < 8 && H * splits * 2 <= 2 * sm_count()) splits *= 2;  // up to ~2 CTAs per SM, at most 8 per head
  AttnFusedParams p{(const __half *)vqk_f16, inv_freq, pos_dev, (__half *)k_cache_f16, (__half *)v_cache_f16, (__half *)out_f16,
                    H, max_seq, kv_stride, scale, KvPages{page_table, page_table ? page_shift_of(page_rows) : 0}};
  const size_t smem = ((size_t)16 * ATT_D + ATT_D + 2 * 8) * sizeof(float);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(H * splits, 1, 1);
  cfg.blockDim = dim3(ATT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  AB200_CUDA(cudaLaunchKernelEx(&cfg, attention_fused_kernel, p));
  return AB200_OK;
}

extern "C" int ab200_attention_fused(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev, void *k_cache_f16,
                                     void *v_cache_f16, void *out_f16, int H, int D, long kv_stride, int max_seq, float scale,
                                     void *stream) {
  return attention_fused_impl(vqk_f16, inv_freq, pos_dev, k_cache_f16, v_cache_f16, out_f16, H, D, kv_stride, max_seq, scale, nullptr, 0, stream);
}

extern "C" int ab200_attention_fused_paged(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev, void *k_cache_f16,
                                           void *v_cache_f16, void *out_f16, int H, int D, long kv_stride, int max_seq, float scale,
                                           const int32_t *page_table, int page_rows, void *stream) {
  if (!page_table) return fail(AB200_EINVAL, "attention_fused_paged: null page table");
  return attention_fused_impl(vqk_f16, inv_freq, pos_dev, k_cache_f16, v_cache_f16, out_f16, H, D, kv_stride, max_seq, scale, page_table, page_rows, stream);
}

// Causal attention of `rows` consecutive tokens over a cache that already holds their keys and
// values: query row r (position *pos0_dev + r) attends cache rows 0 .. *pos0_dev + r.  The batched
// form of ab200_attention_decode (grid = heads x rows).
static int attention_prefill_impl(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16, void *out_f16, const int32_t *pos0_dev,
                                  int rows, int max_seq, int H, int D, long kv_stride, float scale, const int32_t *page_table, int page_rows,
                                  void *stream) {
  clear_error();
  AB200_REQUIRE(page_table == nullptr || page_shift_of(page_rows) >= 0, "attention_prefill: page_rows=%d must be a power of two", page_rows);
  AB200_REQUIRE(q_f16 && k_cache_f16 && v_cache_f16 && out_f16 && pos0_dev && rows > 0 && rows <= 65535, "attention_prefill: bad argument");
  AB200_REQUIRE(D == ATT_D, "attention_prefill: head size %d is not the built size %d", D, ATT_D);
  AB200_REQUIRE(H > 0 && max_seq > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0, "attention_prefill: bad shape H=%d max_seq=%d kv_stride=%ld", H, max_seq, kv_stride);
  AB200_REQUIRE(aligned16(q_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16) && aligned16(out_f16), "attention_prefill: pointers must be 16-byte aligned");
  const size_t smem = ((size_t)max_seq + 16 * ATT_D) * sizeof(float);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "attention_prefill: max_seq=%d exceeds the shared-memory score buffer", max_seq);
  if (smem > 48 * 1024) AB200_CUDA(cudaFuncSetAttribute(attention_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  attention_decode_kernel<__half><<<dim3(H, rows), ATT_THREADS, smem, (cudaStream_t)stream>>>(
      (const __half *)q_f16, (const __half *)k_cache_f16, (const __half *)v_cache_f16, (__half *)out_f16, pos0_dev, 1, max_seq, kv_stride, scale,
      KvPages{page_table, page_table ? page_shift_of(page_rows) : 0});
  AB200_CHECK_LAUNCH("attention_prefill");
  return AB200_OK;
}

extern "C" int ab200_attention_prefill(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16, void *out_f16, const int32_t *pos0_dev,
                                       int rows, int max_seq, int H, int D, long kv_stride, float scale, void *stream) {
  return attention_prefill_impl(q_f16, k_cache_f16, v_cache_f16, out_f16, pos0_dev, rows, max_seq, H, D, kv_stride, scale, nullptr, 0, stream);
}

extern "C" int ab200_attention_prefill_paged(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16, void *out_f16,
                                             const int32_t *pos0_dev, int rows, int max_seq, int H, int D, long kv_stride, float scale,
                                             const int32_t *page_table, int page_rows, void *stream) {
  if (!page_table) return fail(AB200_EINVAL, "attention_prefill_paged: null page table");
  return attention_prefill_impl(q_f16, k_cache_f16, v_cache_f16, out_f16, pos0_dev, rows, max_seq, H, D, kv_stride, scale, page_table, page_rows, stream);
}

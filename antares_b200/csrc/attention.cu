// Single-query (decode) attention over an fp16 KV cache, and the dense fp16 classifier GEMV.
// Both are HBM-bound streams: 16-byte loads, fp32 math, warp-shuffle reductions.
#include <math_constants.h>

#include "common.cuh"

namespace ab200 {

constexpr int ATT_THREADS = 256;
constexpr int ATT_D = 128;

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
__global__ void __launch_bounds__(ATT_THREADS) attention_decode_kernel(const __half *__restrict__ q, const __half *__restrict__ kc,
                                                                      const __half *__restrict__ vc, __half *__restrict__ out,
                                                                      const int32_t *__restrict__ seq_len_dev, int seq_len_add,
                                                                      int max_seq, long kv_stride, float scale) {
  extern __shared__ __align__(16) float att_smem[];
  float *p = att_smem;                // [max_seq]
  float *red = att_smem + max_seq;    // [16][128]
  __shared__ float sh[32];
  const int h = blockIdx.x;
  int S = *seq_len_dev + seq_len_add;
  S = S < 0 ? 0 : (S > max_seq ? max_seq : S);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 15, hw = lane >> 4;

  float qf[8];
  h8_to_f8(*reinterpret_cast<const uint4 *>(q + (size_t)h * ATT_D + sub * 8), qf);
  const __half *kh = kc + (size_t)h * ATT_D + sub * 8;
  float mx = -CUDART_INF_F;
  for (int s0 = warp * 2; s0 < S; s0 += 2 * (ATT_THREADS / 32)) {
    const int s = s0 + hw;
    float dot = 0.f;
    if (s < S) {
      float kf[8];
      h8_to_f8(ldg_stream_v4(kh + (size_t)s * kv_stride), kf);
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
  const __half *vh = vc + (size_t)h * ATT_D + dchunk * 8;
  for (int s = sgroup; s < S; s += 16) {
    float vf[8];
    h8_to_f8(ldg_stream_v4(vh + (size_t)s * kv_stride), vf);
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
    out[(size_t)h * ATT_D + threadIdx.x] = __float2half_rn(S > 0 ? t / sum : 0.f);
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
                                      float scale, void *stream) {
  clear_error();
  AB200_REQUIRE(q_f16 && k_cache_f16 && v_cache_f16 && out_f16 && seq_len_dev, "attention_decode: null pointer");
  AB200_REQUIRE(D == ATT_D, "attention_decode: head size %d is not the built size %d", D, ATT_D);
  AB200_REQUIRE(H > 0 && max_seq > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0, "attention_decode: bad shape H=%d max_seq=%d kv_stride=%ld", H, max_seq, kv_stride);
  AB200_REQUIRE(aligned16(q_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16) && aligned16(out_f16),
                "attention_decode: pointers must be 16-byte aligned");
  const size_t smem = ((size_t)max_seq + 16 * ATT_D) * sizeof(float);
  if (smem > 200 * 1024) return fail(AB200_EUNSUPPORTED, "attention_decode: max_seq=%d exceeds the shared-memory score buffer", max_seq);
  if (smem > 48 * 1024)
    AB200_CUDA(cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  attention_decode_kernel<<<H, ATT_THREADS, smem, (cudaStream_t)stream>>>((const __half *)q_f16, (const __half *)k_cache_f16,
                                                                         (const __half *)v_cache_f16, (__half *)out_f16, seq_len_dev,
                                                                         seq_len_add, max_seq, kv_stride, scale);
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

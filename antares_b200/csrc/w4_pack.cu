// int4 packing utilities: unpack / pack / dequantise.  HBM-bound elementwise kernels; each
// thread owns one packed word (one column, 8 consecutive k) so that reads of qweight and
// writes of each output row are coalesced along N.
#include "common.cuh"

namespace ab200 {

// IR statement 1, samples/05_llama2_7b_int4.py:136.
__global__ void w4_unpack_kernel(const int32_t *__restrict__ qw, int Kp, int N, uint8_t *__restrict__ out) {
  const size_t total = (size_t)Kp * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / N, n = i % N;
    const uint32_t w = (uint32_t)qw[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) out[(r * 8 + j) * N + n] = (uint8_t)((w >> (4 * j)) & 15u);
  }
}

__global__ void w4_pack_kernel(const uint8_t *__restrict__ q, int Kp, int N, int32_t *__restrict__ out) {
  const size_t total = (size_t)Kp * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / N, n = i % N;
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) w |= (uint32_t)(q[(r * 8 + j) * N + n] & 15u) << (4 * j);
    out[i] = (int32_t)w;
  }
}

// IR statements 1-2, samples/05_llama2_7b_int4.py:136-137, in the scales' dtype:
// fp16: one IEEE fp16 multiply of scale and the exact fp16 value q-8; fp32: one fp32 multiply.
template <typename T>
__global__ void w4_dequant_kernel(const int32_t *__restrict__ qw, const T *__restrict__ scales, int Kp, int N,
                                  int group, T *__restrict__ out) {
  const size_t total = (size_t)Kp * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / N, n = i % N;
    const uint32_t w = (uint32_t)qw[i];
    const T sc = scales[((r * 8) / group) * N + n];  // group % 8 == 0: one scale per word
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int q = (int)((w >> (4 * j)) & 15u) - 8;
      T v;
      if (sizeof(T) == 2) v = (T)__hmul((__half)sc, __int2half_rn(q));
      else v = (T)((float)sc * (float)q);
      out[(r * 8 + j) * N + n] = v;
    }
  }
}

static int grid_for(size_t total, int threads) {
  size_t blocks = (total + threads - 1) / threads;
  const size_t cap = (size_t)sm_count() * 16;
  return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_w4_unpack(const int32_t *qweight, int K, int N, uint8_t *q_out, void *stream) {
  clear_error();
  AB200_REQUIRE(qweight && q_out, "w4_unpack: null pointer");
  AB200_REQUIRE(K > 0 && K % 8 == 0 && N > 0, "w4_unpack: K=%d must be a positive multiple of 8, N=%d positive", K, N);
  const size_t total = (size_t)(K / 8) * N;
  w4_unpack_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(qweight, K / 8, N, q_out);
  AB200_CHECK_LAUNCH("w4_unpack");
  return AB200_OK;
}

extern "C" int ab200_w4_pack(const uint8_t *q, int K, int N, int32_t *qweight_out, void *stream) {
  clear_error();
  AB200_REQUIRE(q && qweight_out, "w4_pack: null pointer");
  AB200_REQUIRE(K > 0 && K % 8 == 0 && N > 0, "w4_pack: K=%d must be a positive multiple of 8, N=%d positive", K, N);
  const size_t total = (size_t)(K / 8) * N;
  w4_pack_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(q, K / 8, N, qweight_out);
  AB200_CHECK_LAUNCH("w4_pack");
  return AB200_OK;
}

extern "C" int ab200_w4_dequant(const int32_t *qweight, const void *scales, int K, int N, int group, int dtype,
                                void *w_out, void *stream) {
  clear_error();
  AB200_REQUIRE(qweight && scales && w_out, "w4_dequant: null pointer");
  AB200_REQUIRE(K > 0 && K % 8 == 0 && N > 0, "w4_dequant: K=%d must be a positive multiple of 8, N=%d positive", K, N);
  AB200_REQUIRE(group > 0 && group % 8 == 0 && K % group == 0, "w4_dequant: group=%d must be a multiple of 8 dividing K=%d", group, K);
  const size_t total = (size_t)(K / 8) * N;
  const int grid = grid_for(total, 256);
  if (dtype == AB200_F16)
    w4_dequant_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(qweight, (const __half *)scales, K / 8, N, group, (__half *)w_out);
  else if (dtype == AB200_F32)
    w4_dequant_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(qweight, (const float *)scales, K / 8, N, group, (float *)w_out);
  else
    return fail(AB200_EINVAL, "w4_dequant: unknown dtype %d", dtype);
  AB200_CHECK_LAUNCH("w4_dequant");
  return AB200_OK;
}

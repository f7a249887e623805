// Elementwise and row-reduction operators around the W4A16 contraction, plus the small
// device-side glue kernels of the decode step.  All are single-pass and HBM-bound:
// 128-bit loads, fp32 math, rows kept in registers between the reduction and the scaling pass.
#include <math_constants.h>

#include "common.cuh"

namespace ab200 {

constexpr int ROW_THREADS = 256;
constexpr int ROW_MAX_VEC = 8;  // 8 x 8 elements x 256 threads = 16384 columns

__device__ __forceinline__ float block_sum(float v, float *sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < (int)(blockDim.x >> 5)) ? sh[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_max(float v, float *sh) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < (int)(blockDim.x >> 5)) ? sh[lane] : -CUDART_INF_F;
  t = warp_max(t);
  __syncthreads();
  return t;
}

// 8 consecutive elements of a row as fp32, from fp16 or fp32 storage.
template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4 *>(p);
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(u2h2(u[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8(T *p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<__half>(__half *p, const float (&f)[8]) {
  uint4 v;
  v.x = h22u(__floats2half2_rn(f[0], f[1]));
  v.y = h22u(__floats2half2_rn(f[2], f[3]));
  v.z = h22u(__floats2half2_rn(f[4], f[5]));
  v.w = h22u(__floats2half2_rn(f[6], f[7]));
  *reinterpret_cast<uint4 *>(p) = v;
}
template <>
__device__ __forceinline__ void store8<float>(float *p, const float (&f)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// ---- sigmoid: README.md:66, out = 1 - 1/(1 + exp(x)) -----------------------------------------
__device__ __forceinline__ float sigmoid_readme(float x) { return 1.0f - 1.0f / (1.0f + expf(x)); }

template <typename T>
__global__ void sigmoid_kernel(const T *__restrict__ x, T *__restrict__ out, size_t n) {
  const size_t nvec = n / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    load8<T>(x + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = sigmoid_readme(f[j]);
    store8<T>(out + i * 8, f);
  }
  if (blockIdx.x == 0) {
    for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) out[i] = (T)sigmoid_readme((float)x[i]);
  }
}

// ---- RMSNorm -----------------------------------------------------------------------------------
// Persistent CTAs walk the rows with a stride of the grid; a row stays in registers between the sum
// of squares and the scaling, and the NEXT row's loads are issued before the current row is reduced,
// so the global-load latency of one row hides behind the reduction and the stores of the one before.
// The norm weights of a thread's columns are loaded once.  VEC = 8-element vectors per thread.
template <typename T, int VEC>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_rows_kernel(const T *__restrict__ x, const __half *__restrict__ w,
                                                                  __half *__restrict__ out, int rows, int cols, float eps) {
  __shared__ float sh[32];
  const int nvec = cols / 8;
  float wf[VEC][8];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    const int i = v * ROW_THREADS + threadIdx.x;
    if (i < nvec) load8<__half>(w + (size_t)i * 8, wf[v]);
  }
  float cur[VEC][8], nxt[VEC][8];
  auto load_row = [&](int row, float (&f)[VEC][8]) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int i = v * ROW_THREADS + threadIdx.x;
      if (i < nvec) load8<T>(x + (size_t)row * cols + (size_t)i * 8, f[v]);
    }
  };
  int row = blockIdx.x;
  if (row < rows) load_row(row, cur);
  for (; row < rows; row += gridDim.x) {
    const int next = row + gridDim.x;
    if (next < rows) load_row(next, nxt);
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int i = v * ROW_THREADS + threadIdx.x;
      if (i < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += cur[v][j] * cur[v][j];
      }
    }
    ss = block_sum(ss, sh);
    const float rs = rsqrtf(ss * (1.0f / (float)cols) + eps);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int i = v * ROW_THREADS + threadIdx.x;
      if (i < nvec) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = cur[v][j] * rs * wf[v][j];
        store8<__half>(out + (size_t)row * cols + (size_t)i * 8, g);
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v)
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[v][j] = nxt[v][j];
  }
}

// The AutoRT call form (samples/05_llama2_7b_int4.py:128-131): the caller supplies vsum.
template <typename T>
__global__ void rmsnorm_vsum_kernel(const T *__restrict__ x, const float *__restrict__ vsum, const T *__restrict__ w,
                                    T *__restrict__ out, size_t n, float inv_n, float eps) {
  const float rs = rsqrtf(vsum[0] * inv_n + eps);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = (T)((float)x[i] * rs * (float)w[i]);
}

// ---- RoPE (rotate-half) ---------------------------------------------------------------------------
// One CTA per row (= position).  The angle depends on (row, j) only: D/2 threads compute one sine and
// cosine each into shared memory while every thread's first operands are already on their way; then a
// thread owns 8 consecutive j of the first half of some head and their partners in the second half,
// and walks the heads with a stride of the CTA.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) rope_kernel(const T *__restrict__ x, const float *__restrict__ inv_freq,
                                                          const int32_t *__restrict__ pos, T *__restrict__ out,
                                                          int H, int D) {
  __shared__ float sh_c[ROW_THREADS * 8], sh_s[ROW_THREADS * 8];  // D / 2 <= 8 * ROW_THREADS (the host checks D / 16 <= ROW_THREADS)
  const size_t row = blockIdx.x;
  const int half = D / 2, chunks = half / 8;
  const int jc = threadIdx.x % chunks, hslot = threadIdx.x / chunks, hstep = ROW_THREADS / chunks;
  float a[8], b[8];
  const bool active = hslot < hstep && hslot < H;
  if (active) {
    const size_t base0 = (row * H + hslot) * (size_t)D + jc * 8;
    load8<T>(x + base0, a);
    load8<T>(x + base0 + half, b);
  }
  for (int j = threadIdx.x; j < half; j += ROW_THREADS) {
    float sv, cv;
    sincosf((float)pos[row] * inv_freq[j], &sv, &cv);
    sh_s[j] = sv;
    sh_c[j] = cv;
  }
  __syncthreads();
  if (!active) return;
  float c[8], s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c[j] = sh_c[jc * 8 + j];
    s[j] = sh_s[jc * 8 + j];
  }
  for (int h = hslot; h < H; h += hstep) {
    const size_t base = (row * H + h) * (size_t)D + jc * 8;
    float oa[8], ob[8];
    if (h != hslot) {
      load8<T>(x + base, a);
      load8<T>(x + base + half, b);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      oa[j] = a[j] * c[j] - b[j] * s[j];
      ob[j] = b[j] * c[j] + a[j] * s[j];
    }
    store8<T>(out + base, oa);
    store8<T>(out + base + half, ob);
  }
}

// ---- softmax: AntaresIR.md:226 ---------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ out, int cols) {
  __shared__ float sh[32];
  const size_t row = blockIdx.x;
  const int nvec = cols / 8;
  float f[ROW_MAX_VEC][8];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int v = 0; v < ROW_MAX_VEC; ++v) {
    const int i = v * ROW_THREADS + threadIdx.x;
    if (i < nvec) {
      load8<T>(x + row * cols + (size_t)i * 8, f[v]);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[v][j]);
    }
  }
  mx = block_max(mx, sh);
  float sum = 0.f;
#pragma unroll
  for (int v = 0; v < ROW_MAX_VEC; ++v) {
    const int i = v * ROW_THREADS + threadIdx.x;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[v][j] = expf(f[v][j] - mx);
        sum += f[v][j];
      }
    }
  }
  sum = block_sum(sum, sh);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int v = 0; v < ROW_MAX_VEC; ++v) {
    const int i = v * ROW_THREADS + threadIdx.x;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[v][j] *= inv;
      store8<T>(out + row * cols + (size_t)i * 8, f[v]);
    }
  }
}

// ---- decode-step glue ------------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __half *__restrict__ gu, __half *__restrict__ out, int n) {
  gu += (size_t)blockIdx.y * 2 * n;  // one row of [gate | up] per blockIdx.y
  out += (size_t)blockIdx.y * n;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n / 8; i += gridDim.x * blockDim.x) {
    float g[8], u[8];
    load8<__half>(gu + (size_t)i * 8, g);
    load8<__half>(gu + (size_t)n + (size_t)i * 8, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.0f + expf(-g[j])) * u[j];
    store8<__half>(out + (size_t)i * 8, g);
  }
}

__global__ void embed_lookup_kernel(const __half *__restrict__ embed, const int32_t *__restrict__ token,
                                    float *__restrict__ x, int dim, int vocab) {
  int t = token[blockIdx.y];  // one token per blockIdx.y
  x += (size_t)blockIdx.y * dim;
  t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x)
    x[i] = __half2float(embed[(size_t)t * dim + i]);
}

// vqk = [V | Q | K], each H*D.  Rotates Q into q_out and K into cache row pos; copies V to cache row pos.
__global__ void __launch_bounds__(ROW_THREADS) rope_kv_store_kernel(const __half *__restrict__ vqk, const float *__restrict__ inv_freq,
                                                                   const int32_t *__restrict__ pos_dev, __half *__restrict__ q_out,
                                                                   __half *__restrict__ kc, __half *__restrict__ vc, int H, int D,
                                                                   long kv_stride, int max_seq, KvPages pages) {
  const int pos = *pos_dev + (int)blockIdx.x;  // one token per block: positions pos, pos + 1, ...
  if (pos < 0 || pos >= max_seq) return;  // out-of-range step: leave the cache untouched
  const int HD = H * D, half = D / 2, chunks = half / 8;
  vqk += (size_t)blockIdx.x * 3 * HD;
  q_out += (size_t)blockIdx.x * HD;
  const __half *v = vqk, *q = vqk + HD, *k = vqk + 2 * HD;
  const size_t prow = kv_row(pages, pos);
  __half *krow = kc + prow * kv_stride, *vrow = vc + prow * kv_stride;
  for (int i = threadIdx.x; i < HD / 8; i += ROW_THREADS)
    *reinterpret_cast<uint4 *>(vrow + (size_t)i * 8) = *reinterpret_cast<const uint4 *>(v + (size_t)i * 8);
  const int jc = threadIdx.x % chunks, hslot = threadIdx.x / chunks, hstep = ROW_THREADS / chunks;
  float c[8], s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) sincosf((float)pos * inv_freq[jc * 8 + j], &s[j], &c[j]);
  for (int h = hslot; h < H; h += hstep) {
    const size_t base = (size_t)h * D + jc * 8;
    float a[8], b[8], oa[8], ob[8];
    load8<__half>(q + base, a);
    load8<__half>(q + base + half, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) { oa[j] = a[j] * c[j] - b[j] * s[j]; ob[j] = b[j] * c[j] + a[j] * s[j]; }
    store8<__half>(q_out + base, oa);
    store8<__half>(q_out + base + half, ob);
    load8<__half>(k + base, a);
    load8<__half>(k + base + half, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) { oa[j] = a[j] * c[j] - b[j] * s[j]; ob[j] = b[j] * c[j] + a[j] * s[j]; }
    store8<__half>(krow + base, oa);
    store8<__half>(krow + base + half, ob);
  }
}

// x_f32[i] += y_f16[i]: residual update after a prefill GEMM (fp16 output, fp32 residual stream).
__global__ void residual_add_f16_kernel(float *__restrict__ x, const __half *__restrict__ y, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    load8<__half>(y + i * 8, f);
    float4 a = *reinterpret_cast<float4 *>(x + i * 8), b = *reinterpret_cast<float4 *>(x + i * 8 + 4);
    a.x += f[0]; a.y += f[1]; a.z += f[2]; a.w += f[3];
    b.x += f[4]; b.y += f[5]; b.z += f[6]; b.w += f[7];
    *reinterpret_cast<float4 *>(x + i * 8) = a;
    *reinterpret_cast<float4 *>(x + i * 8 + 4) = b;
  }
}

// Greedy token choice and loop bookkeeping in one CTA (first maximum wins, like torch.argmax).
__global__ void __launch_bounds__(1024) greedy_next_kernel(const float *__restrict__ logits, int n, const int32_t *__restrict__ prompt,
                                                          int n_prompt, int32_t *token_dev, int32_t *pos_dev, int32_t *out_tokens,
                                                          int out_cap) {
  __shared__ float sv[32];
  __shared__ int si[32];
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  pdl_launch_dependents();
  pdl_wait();
  // 16-byte loads, four independent ones in flight per thread; ties keep the lowest index
  const int nvec = ((reinterpret_cast<uintptr_t>(logits) & 15u) == 0) ? n / 4 : 0;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = (i < nvec) ? reinterpret_cast<const float4 *>(logits)[i] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = (i0 + u * blockDim.x) * 4;
      const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (e[j] > best || (e[j] == best && i + j < bi)) { best = e[j]; bi = i + j; }
    }
  }
  for (int i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) {
    const float v = logits[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = (lane < (int)(blockDim.x >> 5)) ? sv[lane] : -CUDART_INF_F;
    bi = (lane < (int)(blockDim.x >> 5)) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      const int pos = *pos_dev;
      int next = (bi == 0x7fffffff) ? 0 : bi;
      if (prompt != nullptr && pos + 1 < n_prompt) next = prompt[pos + 1];
      *token_dev = next;
      // the token log holds out_cap ids: past its end nothing is stored and the position stays put,
      // so a step too many cannot write outside the buffer (the host counts steps and raises first)
      if (out_tokens == nullptr) {
        *pos_dev = pos + 1;
      } else if (pos + 1 < out_cap) {
        out_tokens[pos + 1] = next;
        *pos_dev = pos + 1;
      }
    }
  }
}

static int grid1d(size_t work_items, int threads) {
  size_t blocks = (work_items + threads - 1) / threads;
  const size_t cap = (size_t)sm_count() * 8;
  return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_sigmoid(const void *x, void *out, size_t n, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(x && out, "sigmoid: null pointer");
  if (n == 0) return AB200_OK;
  AB200_REQUIRE(aligned16(x) && aligned16(out), "sigmoid: pointers must be 16-byte aligned");
  const int grid = grid1d(n / 8 + 1, 256);
  if (dtype == AB200_F32) sigmoid_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float *)x, (float *)out, n);
  else if (dtype == AB200_F16) sigmoid_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, (__half *)out, n);
  else return fail(AB200_EINVAL, "sigmoid: unknown dtype %d", dtype);
  AB200_CHECK_LAUNCH("sigmoid");
  return AB200_OK;
}

extern "C" int ab200_rmsnorm_vsum(const void *x, const float *vsum, const void *weight, void *out, size_t n,
                                  float inv_n, float eps, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(x && vsum && weight && out, "rmsnorm_vsum: null pointer");
  if (n == 0) return AB200_OK;
  const int grid = grid1d(n, 256);
  if (dtype == AB200_F32)
    rmsnorm_vsum_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float *)x, vsum, (const float *)weight, (float *)out, n, inv_n, eps);
  else if (dtype == AB200_F16)
    rmsnorm_vsum_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, vsum, (const __half *)weight, (__half *)out, n, inv_n, eps);
  else return fail(AB200_EINVAL, "rmsnorm_vsum: unknown dtype %d", dtype);
  AB200_CHECK_LAUNCH("rmsnorm_vsum");
  return AB200_OK;
}

extern "C" int ab200_rmsnorm(const void *x, int x_dtype, const void *weight_f16, void *out_f16, int rows, int cols,
                             float eps, void *stream) {
  clear_error();
  AB200_REQUIRE(x && weight_f16 && out_f16, "rmsnorm: null pointer");
  AB200_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= ROW_THREADS * ROW_MAX_VEC * 8,
                "rmsnorm: cols=%d must be a multiple of 8, at most %d", cols, ROW_THREADS * ROW_MAX_VEC * 8);
  AB200_REQUIRE(aligned16(x) && aligned16(weight_f16) && aligned16(out_f16), "rmsnorm: pointers must be 16-byte aligned");
  if (rows == 0) return AB200_OK;
  AB200_REQUIRE(x_dtype == AB200_F16 || x_dtype == AB200_F32, "rmsnorm: unknown dtype %d", x_dtype);
  const int vec = (cols / 8 + ROW_THREADS - 1) / ROW_THREADS;  // 8-element vectors per thread
  const int cap = sm_count() * (vec <= 2 ? 4 : 2);  // persistent CTAs: about what fits an SM by registers
  const int grid = rows < cap ? rows : cap;
  const cudaStream_t st = (cudaStream_t)stream;
#define AB200_RMS_LAUNCH(T, V) rmsnorm_rows_kernel<T, V><<<grid, ROW_THREADS, 0, st>>>((const T *)x, (const __half *)weight_f16, (__half *)out_f16, rows, cols, eps)
  if (x_dtype == AB200_F16) {
    if (vec <= 1) AB200_RMS_LAUNCH(__half, 1);
    else if (vec <= 2) AB200_RMS_LAUNCH(__half, 2);
    else if (vec <= 4) AB200_RMS_LAUNCH(__half, 4);
    else AB200_RMS_LAUNCH(__half, 8);
  } else {
    if (vec <= 1) AB200_RMS_LAUNCH(float, 1);
    else if (vec <= 2) AB200_RMS_LAUNCH(float, 2);
    else if (vec <= 4) AB200_RMS_LAUNCH(float, 4);
    else AB200_RMS_LAUNCH(float, 8);
  }
#undef AB200_RMS_LAUNCH
  AB200_CHECK_LAUNCH("rmsnorm");
  return AB200_OK;
}

extern "C" int ab200_rope(const void *x_f16, const float *inv_freq, const int32_t *pos, void *out_f16, int rows, int H,
                          int D, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(x_f16 && inv_freq && pos && out_f16, "rope: null pointer");
  AB200_REQUIRE(D > 0 && D % 16 == 0 && D / 16 <= ROW_THREADS && H > 0 && rows >= 0, "rope: D=%d must be a multiple of 16 (at most %d), H=%d positive", D, ROW_THREADS * 16, H);
  AB200_REQUIRE(aligned16(x_f16) && aligned16(out_f16), "rope: pointers must be 16-byte aligned");
  if (rows == 0) return AB200_OK;
  if (dtype == AB200_F16) rope_kernel<__half><<<rows, ROW_THREADS, 0, (cudaStream_t)stream>>>((const __half *)x_f16, inv_freq, pos, (__half *)out_f16, H, D);
  else if (dtype == AB200_F32) rope_kernel<float><<<rows, ROW_THREADS, 0, (cudaStream_t)stream>>>((const float *)x_f16, inv_freq, pos, (float *)out_f16, H, D);
  else return fail(AB200_EINVAL, "rope: unknown dtype %d", dtype);
  AB200_CHECK_LAUNCH("rope");
  return AB200_OK;
}

extern "C" int ab200_softmax(const void *x, void *out, int rows, int cols, int dtype, void *stream) {
  clear_error();
  AB200_REQUIRE(x && out, "softmax: null pointer");
  AB200_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= ROW_THREADS * ROW_MAX_VEC * 8,
                "softmax: cols=%d must be a multiple of 8, at most %d", cols, ROW_THREADS * ROW_MAX_VEC * 8);
  AB200_REQUIRE(aligned16(x) && aligned16(out), "softmax: pointers must be 16-byte aligned");
  if (rows == 0) return AB200_OK;
  if (dtype == AB200_F16) softmax_rows_kernel<__half><<<rows, ROW_THREADS, 0, (cudaStream_t)stream>>>((const __half *)x, (__half *)out, cols);
  else if (dtype == AB200_F32) softmax_rows_kernel<float><<<rows, ROW_THREADS, 0, (cudaStream_t)stream>>>((const float *)x, (float *)out, cols);
  else return fail(AB200_EINVAL, "softmax: unknown dtype %d", dtype);
  AB200_CHECK_LAUNCH("softmax");
  return AB200_OK;
}

extern "C" int ab200_silu_mul(const void *gate_up_f16, void *out_f16, int n, void *stream) {
  clear_error();
  AB200_REQUIRE(gate_up_f16 && out_f16, "silu_mul: null pointer");
  AB200_REQUIRE(n > 0 && n % 8 == 0, "silu_mul: n=%d must be a positive multiple of 8", n);
  AB200_REQUIRE(aligned16(gate_up_f16) && aligned16(out_f16), "silu_mul: pointers must be 16-byte aligned");
  silu_mul_kernel<<<grid1d(n / 8, 128), 128, 0, (cudaStream_t)stream>>>((const __half *)gate_up_f16, (__half *)out_f16, n);
  AB200_CHECK_LAUNCH("silu_mul");
  return AB200_OK;
}

extern "C" int ab200_embed_lookup(const void *embed_f16, const int32_t *token_dev, float *x_f32, int dim, int vocab,
                                  void *stream) {
  clear_error();
  AB200_REQUIRE(embed_f16 && token_dev && x_f32 && dim > 0 && vocab > 0, "embed_lookup: bad argument");
  embed_lookup_kernel<<<grid1d(dim, 256), 256, 0, (cudaStream_t)stream>>>((const __half *)embed_f16, token_dev, x_f32, dim, vocab);
  AB200_CHECK_LAUNCH("embed_lookup");
  return AB200_OK;
}

extern "C" int ab200_rope_kv_store(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev, void *q_out_f16,
                                   void *k_cache_f16, void *v_cache_f16, int H, int D, long kv_stride, int max_seq,
                                   void *stream) {
  clear_error();
  AB200_REQUIRE(vqk_f16 && inv_freq && pos_dev && q_out_f16 && k_cache_f16 && v_cache_f16, "rope_kv_store: null pointer");
  AB200_REQUIRE(D > 0 && D % 16 == 0 && D / 16 <= ROW_THREADS && H > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0,
                "rope_kv_store: bad shape H=%d D=%d kv_stride=%ld", H, D, kv_stride);
  AB200_REQUIRE(aligned16(vqk_f16) && aligned16(q_out_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16),
                "rope_kv_store: pointers must be 16-byte aligned");
  rope_kv_store_kernel<<<1, ROW_THREADS, 0, (cudaStream_t)stream>>>((const __half *)vqk_f16, inv_freq, pos_dev, (__half *)q_out_f16,
                                                                  (__half *)k_cache_f16, (__half *)v_cache_f16, H, D, kv_stride, max_seq, KvPages{nullptr, 0});
  AB200_CHECK_LAUNCH("rope_kv_store");
  return AB200_OK;
}

extern "C" int ab200_greedy_next(const float *logits_f32, int n, const int32_t *prompt, int n_prompt, int32_t *token_dev,
                                 int32_t *pos_dev, int32_t *out_tokens, int out_cap, void *stream) {
  clear_error();
  AB200_REQUIRE(logits_f32 && token_dev && pos_dev && n > 0, "greedy_next: bad argument");
  AB200_REQUIRE(out_tokens == nullptr || out_cap > 0, "greedy_next: the token log needs a positive capacity");
  greedy_next_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(logits_f32, n, prompt, n_prompt, token_dev, pos_dev, out_tokens, out_cap);
  AB200_CHECK_LAUNCH("greedy_next");
  return AB200_OK;
}

// ---- batched (prefill) forms of the decode-step glue: one row per prompt token ---------------------

extern "C" int ab200_embed_rows(const void *embed_f16, const int32_t *tokens_dev, float *x_f32, int rows, int dim, int vocab, void *stream) {
  clear_error();
  AB200_REQUIRE(embed_f16 && tokens_dev && x_f32 && rows > 0 && rows <= 65535 && dim > 0 && vocab > 0, "embed_rows: bad argument");
  embed_lookup_kernel<<<dim3(grid1d(dim, 256), rows), 256, 0, (cudaStream_t)stream>>>((const __half *)embed_f16, tokens_dev, x_f32, dim, vocab);
  AB200_CHECK_LAUNCH("embed_rows");
  return AB200_OK;
}

static int rope_kv_store_rows_impl(const void *vqk_f16, const float *inv_freq, const int32_t *pos0_dev, void *q_out_f16, void *k_cache_f16,
                                   void *v_cache_f16, int rows, int H, int D, long kv_stride, int max_seq, const int32_t *page_table,
                                   int page_rows, void *stream) {
  clear_error();
  AB200_REQUIRE(vqk_f16 && inv_freq && pos0_dev && q_out_f16 && k_cache_f16 && v_cache_f16 && rows > 0, "rope_kv_store_rows: bad argument");
  AB200_REQUIRE(D > 0 && D % 16 == 0 && D / 16 <= ROW_THREADS && H > 0 && kv_stride >= (long)H * D && kv_stride % 8 == 0,
                "rope_kv_store_rows: bad shape H=%d D=%d kv_stride=%ld", H, D, kv_stride);
  AB200_REQUIRE(aligned16(vqk_f16) && aligned16(q_out_f16) && aligned16(k_cache_f16) && aligned16(v_cache_f16),
                "rope_kv_store_rows: pointers must be 16-byte aligned");
  int shift = 0;
  if (page_table) {
    while ((1 << shift) < page_rows) ++shift;
    AB200_REQUIRE(page_rows > 0 && (1 << shift) == page_rows, "rope_kv_store_rows: page_rows=%d must be a power of two", page_rows);
  }
  rope_kv_store_kernel<<<rows, ROW_THREADS, 0, (cudaStream_t)stream>>>((const __half *)vqk_f16, inv_freq, pos0_dev, (__half *)q_out_f16,
                                                                     (__half *)k_cache_f16, (__half *)v_cache_f16, H, D, kv_stride, max_seq,
                                                                     KvPages{page_table, shift});
  AB200_CHECK_LAUNCH("rope_kv_store_rows");
  return AB200_OK;
}

extern "C" int ab200_rope_kv_store_rows(const void *vqk_f16, const float *inv_freq, const int32_t *pos0_dev, void *q_out_f16, void *k_cache_f16,
                                        void *v_cache_f16, int rows, int H, int D, long kv_stride, int max_seq, void *stream) {
  return rope_kv_store_rows_impl(vqk_f16, inv_freq, pos0_dev, q_out_f16, k_cache_f16, v_cache_f16, rows, H, D, kv_stride, max_seq, nullptr, 0, stream);
}

extern "C" int ab200_rope_kv_store_rows_paged(const void *vqk_f16, const float *inv_freq, const int32_t *pos0_dev, void *q_out_f16,
                                              void *k_cache_f16, void *v_cache_f16, int rows, int H, int D, long kv_stride, int max_seq,
                                              const int32_t *page_table, int page_rows, void *stream) {
  if (!page_table) return fail(AB200_EINVAL, "rope_kv_store_rows_paged: null page table");
  return rope_kv_store_rows_impl(vqk_f16, inv_freq, pos0_dev, q_out_f16, k_cache_f16, v_cache_f16, rows, H, D, kv_stride, max_seq, page_table, page_rows,
                                 stream);
}

extern "C" int ab200_silu_mul_rows(const void *gate_up_f16, void *out_f16, int rows, int n, void *stream) {
  clear_error();
  AB200_REQUIRE(gate_up_f16 && out_f16 && rows > 0 && rows <= 65535 && n > 0 && n % 8 == 0, "silu_mul_rows: n=%d must be a positive multiple of 8", n);
  AB200_REQUIRE(aligned16(gate_up_f16) && aligned16(out_f16), "silu_mul_rows: pointers must be 16-byte aligned");
  silu_mul_kernel<<<dim3(grid1d(n / 8, 128), rows), 128, 0, (cudaStream_t)stream>>>((const __half *)gate_up_f16, (__half *)out_f16, n);
  AB200_CHECK_LAUNCH("silu_mul_rows");
  return AB200_OK;
}

extern "C" int ab200_residual_add_f16(float *x_f32, const void *y_f16, size_t n, void *stream) {
  clear_error();
  AB200_REQUIRE(x_f32 && y_f16 && n > 0 && n % 8 == 0, "residual_add_f16: n must be a positive multiple of 8");
  AB200_REQUIRE(aligned16(x_f32) && aligned16(y_f16), "residual_add_f16: pointers must be 16-byte aligned");
  residual_add_f16_kernel<<<grid1d(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(x_f32, (const __half *)y_f16, n / 8);
  AB200_CHECK_LAUNCH("residual_add_f16");
  return AB200_OK;
}

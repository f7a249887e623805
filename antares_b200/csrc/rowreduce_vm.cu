// Row-reduction template for multi-statement Antares-IR programs outside the named operator family:
// a chain of row reductions followed by one map statement over the same [rows, cols] index space,
//   t0[N] >=! f0(x[N, C]);  t1[N] +=! f1(x[N, C], t0[N]);  out[N, C] = g(x[N, C], t0[N], t1[N])
// (softmax, AntaresIR.md:226; layernorm, AntaresIR.md:232).  The reference compiles each statement
// into its own generated kernel (lang/einstein_v2.py:297-578 -> antares/default_codegen.py); here one
// kernel runs all stages of a row back to back: every stage's expression is a small stack program
// (the same operation set as the element-wise interpreter, plus "row value of an earlier stage",
// "column vector" and "number of columns"), evaluated per element in fp32; a reduction stage folds
// the values of a row with + / max / min (warp shuffles, one shared-memory hop, fixed order, so
// results are bitwise repeatable), the final stage writes the output.  The row stays in L1/L2
// between stages, so HBM sees each input once.
#include <math_constants.h>

#include "common.cuh"

namespace ab200 {

constexpr int RV_MAX_STAGES = 4, RV_MAX_OPS = 48, RV_MAX_CONSTS = 16, RV_MAX_MAT = 4, RV_MAX_COL = 4, RV_MAX_STACK = 8;
constexpr int RV_THREADS = 256;

// operation codes: 0-21 as in the element-wise interpreter (eltwise_vm.cu), then
enum { RV_IN = 0, RV_CONST = 1, RV_ADD = 2, RV_SUB, RV_MUL, RV_DIV, RV_NEG, RV_EXP, RV_LOG, RV_SQRT, RV_RSQRT, RV_TANH, RV_ERF, RV_SIN, RV_COS,
       RV_ABS, RV_FLOOR, RV_CEIL, RV_MAX, RV_MIN, RV_POW, RV_SIGMOID, RV_ROW = 22, RV_COL = 23, RV_COLLEN = 24, RV_OP_COUNT };
enum { RV_MAP = 0, RV_SUM = 1, RV_RMAX = 2, RV_RMIN = 3 };

struct RowProgram {
  const void *mat[RV_MAX_MAT];  // [rows, cols]
  const void *col[RV_MAX_COL];  // [cols]
  void *out;                    // [rows, cols]
  float cst[RV_MAX_CONSTS];
  unsigned char op[RV_MAX_STAGES][RV_MAX_OPS], arg[RV_MAX_STAGES][RV_MAX_OPS];
  unsigned char n_ops[RV_MAX_STAGES], reduce[RV_MAX_STAGES];
  unsigned char mat_f16[RV_MAX_MAT], col_f16[RV_MAX_COL];
  int n_stages, out_f16, rows, cols;
};

__device__ __forceinline__ float rv_load(const void *p, bool f16, size_t i) {
  return f16 ? __half2float(reinterpret_cast<const __half *>(p)[i]) : reinterpret_cast<const float *>(p)[i];
}

__global__ void __launch_bounds__(RV_THREADS) rowreduce_vm_kernel(const __grid_constant__ RowProgram p) {
  __shared__ float st[RV_MAX_STACK][RV_THREADS];
  __shared__ float warp_part[RV_THREADS / 32];
  __shared__ float rowval[RV_MAX_STAGES];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const size_t base = (size_t)row * p.cols;
    for (int s = 0; s < p.n_stages; ++s) {
      const int kind = p.reduce[s];
      float acc = kind == RV_RMAX ? -CUDART_INF_F : kind == RV_RMIN ? CUDART_INF_F : 0.f;
      for (int c = threadIdx.x; c < p.cols; c += RV_THREADS) {
        // the top of the operand stack stays in a register; shared memory holds what is underneath it
        int sp = 0;
        float top = 0.f;
        for (int k = 0; k < p.n_ops[s]; ++k) {
          const int op = p.op[s][k], arg = p.arg[s][k];
          if (op <= RV_CONST || op >= RV_ROW) {
            if (k > 0) st[sp++][threadIdx.x] = top;
            if (op == RV_IN) top = rv_load(p.mat[arg], p.mat_f16[arg], base + c);
            else if (op == RV_CONST) top = p.cst[arg];
            else if (op == RV_ROW) top = rowval[arg];
            else if (op == RV_COL) top = rv_load(p.col[arg], p.col_f16[arg], c);
            else top = (float)p.cols;
          } else if (op <= RV_DIV || (op >= RV_MAX && op <= RV_POW)) {
            const float b = top, a = st[--sp][threadIdx.x];
            switch (op) {
              case RV_ADD: top = a + b; break;
              case RV_SUB: top = a - b; break;
              case RV_MUL: top = a * b; break;
              case RV_DIV: top = a / b; break;
              case RV_MAX: top = fmaxf(a, b); break;
              case RV_MIN: top = fminf(a, b); break;
              default: top = powf(a, b); break;
            }
          } else {
            const float a = top;
            switch (op) {
              case RV_NEG: top = -a; break;
              case RV_EXP: top = expf(a); break;
              case RV_LOG: top = logf(a); break;
              case RV_SQRT: top = sqrtf(a); break;
              case RV_RSQRT: top = rsqrtf(a); break;
              case RV_TANH: top = tanhf(a); break;
              case RV_ERF: top = erff(a); break;
              case RV_SIN: top = sinf(a); break;
              case RV_COS: top = cosf(a); break;
              case RV_ABS: top = fabsf(a); break;
              case RV_FLOOR: top = floorf(a); break;
              case RV_CEIL: top = ceilf(a); break;
              default: top = 1.0f / (1.0f + expf(-a)); break;  // RV_SIGMOID
            }
          }
        }
        if (kind == RV_MAP) {
          if (p.out_f16) reinterpret_cast<__half *>(p.out)[base + c] = __float2half_rn(top);
          else reinterpret_cast<float *>(p.out)[base + c] = top;
        } else if (kind == RV_SUM) {
          acc += top;
        } else if (kind == RV_RMAX) {
          acc = fmaxf(acc, top);
        } else {
          acc = fminf(acc, top);
        }
      }
      if (kind != RV_MAP) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float other = __shfl_xor_sync(0xffffffffu, acc, o);
          acc = kind == RV_SUM ? acc + other : kind == RV_RMAX ? fmaxf(acc, other) : fminf(acc, other);
        }
        if (lane == 0) warp_part[warp] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
          float r = warp_part[0];
          for (int w = 1; w < RV_THREADS / 32; ++w) r = kind == RV_SUM ? r + warp_part[w] : kind == RV_RMAX ? fmaxf(r, warp_part[w]) : fminf(r, warp_part[w]);
          rowval[s] = r;
        }
        __syncthreads();
      }
    }
    __syncthreads();  // rowval and warp_part are reused by the next row
  }
}

}  // namespace ab200

using namespace ab200;

extern "C" int ab200_rowreduce_vm(const unsigned char *ops_host, const unsigned char *args_host, const int *stage_len_host,
                                  const int *stage_reduce_host, int n_stages, const float *consts_host, int n_consts,
                                  const void *const *mat_inputs_host, const int *mat_dtypes_host, int n_mat, const void *const *col_inputs_host,
                                  const int *col_dtypes_host, int n_col, void *out, int out_dtype, int rows, int cols, void *stream) {
  clear_error();
  AB200_REQUIRE(ops_host && args_host && stage_len_host && stage_reduce_host && out, "rowreduce_vm: null pointer");
  AB200_REQUIRE(n_stages >= 1 && n_stages <= RV_MAX_STAGES, "rowreduce_vm: %d stages (1..%d)", n_stages, RV_MAX_STAGES);
  AB200_REQUIRE(n_consts >= 0 && n_consts <= RV_MAX_CONSTS && (n_consts == 0 || consts_host), "rowreduce_vm: %d constants (at most %d)", n_consts, RV_MAX_CONSTS);
  AB200_REQUIRE(n_mat >= 1 && n_mat <= RV_MAX_MAT && mat_inputs_host && mat_dtypes_host, "rowreduce_vm: %d [rows, cols] inputs (1..%d)", n_mat, RV_MAX_MAT);
  AB200_REQUIRE(n_col >= 0 && n_col <= RV_MAX_COL && (n_col == 0 || (col_inputs_host && col_dtypes_host)), "rowreduce_vm: %d [cols] inputs (at most %d)", n_col, RV_MAX_COL);
  AB200_REQUIRE(rows > 0 && cols > 0, "rowreduce_vm: rows=%d cols=%d", rows, cols);
  AB200_REQUIRE(out_dtype == AB200_F16 || out_dtype == AB200_F32, "rowreduce_vm: output dtype %d", out_dtype);
  RowProgram p = {};
  for (int i = 0; i < n_mat; ++i) {
    AB200_REQUIRE(mat_inputs_host[i] && (mat_dtypes_host[i] == AB200_F16 || mat_dtypes_host[i] == AB200_F32), "rowreduce_vm: bad matrix input %d", i);
    p.mat[i] = mat_inputs_host[i];
    p.mat_f16[i] = mat_dtypes_host[i] == AB200_F16;
  }
  for (int i = 0; i < n_col; ++i) {
    AB200_REQUIRE(col_inputs_host[i] && (col_dtypes_host[i] == AB200_F16 || col_dtypes_host[i] == AB200_F32), "rowreduce_vm: bad column-vector input %d", i);
    p.col[i] = col_inputs_host[i];
    p.col_f16[i] = col_dtypes_host[i] == AB200_F16;
  }
  for (int i = 0; i < n_consts; ++i) p.cst[i] = consts_host[i];
  // validate every stage on the host: operand indices, stack discipline, stage order
  int off = 0;
  for (int s = 0; s < n_stages; ++s) {
    const int len = stage_len_host[s], kind = stage_reduce_host[s];
    AB200_REQUIRE(len >= 1 && len <= RV_MAX_OPS, "rowreduce_vm: stage %d has %d operations (1..%d)", s, len, RV_MAX_OPS);
    AB200_REQUIRE(kind >= RV_MAP && kind <= RV_RMIN, "rowreduce_vm: stage %d has reduction kind %d", s, kind);
    AB200_REQUIRE((kind == RV_MAP) == (s == n_stages - 1), "rowreduce_vm: the last stage, and only the last, writes the output");
    int depth = 0;
    for (int k = 0; k < len; ++k) {
      const int op = ops_host[off + k], arg = args_host[off + k];
      AB200_REQUIRE(op < RV_OP_COUNT, "rowreduce_vm: unknown operation %d", op);
      if (op <= RV_CONST || op >= RV_ROW) {
        AB200_REQUIRE(op != RV_IN || arg < n_mat, "rowreduce_vm: matrix input index %d out of range", arg);
        AB200_REQUIRE(op != RV_CONST || arg < n_consts, "rowreduce_vm: constant index %d out of range", arg);
        AB200_REQUIRE(op != RV_ROW || arg < s, "rowreduce_vm: stage %d reads the row value of stage %d, which is not earlier", s, arg);
        AB200_REQUIRE(op != RV_COL || arg < n_col, "rowreduce_vm: column-vector index %d out of range", arg);
        ++depth;
      } else if (op <= RV_DIV || (op >= RV_MAX && op <= RV_POW)) {
        AB200_REQUIRE(depth >= 2, "rowreduce_vm: stack underflow in stage %d", s);
        --depth;
      } else {
        AB200_REQUIRE(depth >= 1, "rowreduce_vm: stack underflow in stage %d", s);
      }
      AB200_REQUIRE(depth <= RV_MAX_STACK, "rowreduce_vm: stage %d needs a stack deeper than %d", s, RV_MAX_STACK);
      p.op[s][k] = (unsigned char)op;
      p.arg[s][k] = (unsigned char)arg;
    }
    AB200_REQUIRE(depth == 1, "rowreduce_vm: stage %d leaves %d values on the stack", s, depth);
    p.n_ops[s] = (unsigned char)len;
    p.reduce[s] = (unsigned char)kind;
    off += len;
  }
  p.out = out;
  p.n_stages = n_stages;
  p.out_f16 = out_dtype == AB200_F16;
  p.rows = rows;
  p.cols = cols;
  const int cap = sm_count() * 8;
  rowreduce_vm_kernel<<<rows < cap ? rows : cap, RV_THREADS, 0, (cudaStream_t)stream>>>(p);
  AB200_CHECK_LAUNCH("rowreduce_vm");
  return AB200_OK;
}

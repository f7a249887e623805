// Interpreter for element-wise Antares-IR statements outside the named operator family
// (`out[axes] = expr` with every tensor indexed by the output's axes): the expression arrives as
// a small stack program (antares_b200/ir.py::compile_elementwise) inside the kernel parameters,
// every thread evaluates it for four consecutive elements at a time in fp32.  The reference
// generates a kernel per expression (lang/einstein_v2.py:297-578 -> antares/default_codegen.py);
// here one kernel serves them all, so no compiler is needed at run time.
//
// The top of the operand stack stays in registers, the rest lives in shared memory ([slot][thread]
// float4: conflict-free); the program
// and constants are kernel parameters (uniform loads, one uniform branch per operation, shared
// by the four elements).  Inputs and output may be fp16 or fp32; 16-byte / 8-byte accesses when
// the element count and pointers allow, a scalar tail otherwise.
#include <math_constants.h>

#include "common.cuh"

namespace ab200 {

constexpr int VM_MAX_OPS = 48, VM_MAX_CONSTS = 16, VM_MAX_INPUTS = 8, VM_MAX_STACK = 8;
constexpr int VM_THREADS = 128;

enum VmOp : unsigned char {
  VM_IN = 0, VM_CONST, VM_ADD, VM_SUB, VM_MUL, VM_DIV, VM_NEG, VM_EXP, VM_LOG, VM_SQRT, VM_RSQRT, VM_TANH, VM_ERF, VM_SIN, VM_COS,
  VM_ABS, VM_FLOOR, VM_CEIL, VM_MAX, VM_MIN, VM_POW, VM_SIGMOID, VM_OP_COUNT
};

struct VmProgram {
  const void *in[VM_MAX_INPUTS];
  void *out;
  float cst[VM_MAX_CONSTS];
  unsigned char op[VM_MAX_OPS], arg[VM_MAX_OPS];
  unsigned char in_f16[VM_MAX_INPUTS];
  int n_ops, out_f16;
  size_t n;
};

__device__ __forceinline__ float4 vm_load4(const void *p, bool f16, size_t i, size_t n, bool vec) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) {
    if (f16) {
      const uint2 h = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(p) + i);
      const float2 a = __half22float2(u2h2(h.x)), b = __half22float2(u2h2(h.y));
      v = make_float4(a.x, a.y, b.x, b.y);
    } else {
      v = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i);
    }
  } else {
    float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j < n) e[j] = f16 ? __half2float(reinterpret_cast<const __half *>(p)[i + j]) : reinterpret_cast<const float *>(p)[i + j];
    v = make_float4(e[0], e[1], e[2], e[3]);
  }
  return v;
}

template <typename F>
__device__ __forceinline__ float4 map4(float4 a, F f) { return make_float4(f(a.x), f(a.y), f(a.z), f(a.w)); }
template <typename F>
__device__ __forceinline__ float4 zip4(float4 a, float4 b, F f) { return make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w)); }

__global__ void __launch_bounds__(VM_THREADS) eltwise_vm_kernel(const __grid_constant__ VmProgram p, int vec_ok) {
  __shared__ float4 st[VM_MAX_STACK][VM_THREADS];
  const size_t n4 = (p.n + 3) / 4;
  for (size_t q = (size_t)blockIdx.x * VM_THREADS + threadIdx.x; q < n4; q += (size_t)gridDim.x * VM_THREADS) {
    const size_t i = q * 4;
    const bool vec = vec_ok && (i + 4 <= p.n);
    // the top of the stack stays in registers; shared memory holds what is underneath it
    int sp = 0;  // entries in shared memory
    float4 top = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < p.n_ops; ++k) {
      const int op = p.op[k], arg = p.arg[k];
      if (op <= VM_CONST) {
        if (k > 0) st[sp++][threadIdx.x] = top;
        if (op == VM_IN) {
          top = vm_load4(p.in[arg], p.in_f16[arg], i, p.n, vec);
        } else {
          const float c = p.cst[arg];
          top = make_float4(c, c, c, c);
        }
      } else if (op <= VM_DIV || (op >= VM_MAX && op <= VM_POW)) {
        const float4 b = top, a = st[--sp][threadIdx.x];
        switch (op) {
          case VM_ADD: top = zip4(a, b, [](float x, float y) { return x + y; }); break;
          case VM_SUB: top = zip4(a, b, [](float x, float y) { return x - y; }); break;
          case VM_MUL: top = zip4(a, b, [](float x, float y) { return x * y; }); break;
          case VM_DIV: top = zip4(a, b, [](float x, float y) { return x / y; }); break;
          case VM_MAX: top = zip4(a, b, [](float x, float y) { return fmaxf(x, y); }); break;
          case VM_MIN: top = zip4(a, b, [](float x, float y) { return fminf(x, y); }); break;
          default: top = zip4(a, b, [](float x, float y) { return powf(x, y); }); break;
        }
      } else {
        const float4 a = top;
        switch (op) {
          case VM_NEG: top = map4(a, [](float x) { return -x; }); break;
          case VM_EXP: top = map4(a, [](float x) { return expf(x); }); break;
          case VM_LOG: top = map4(a, [](float x) { return logf(x); }); break;
          case VM_SQRT: top = map4(a, [](float x) { return sqrtf(x); }); break;
          case VM_RSQRT: top = map4(a, [](float x) { return rsqrtf(x); }); break;
          case VM_TANH: top = map4(a, [](float x) { return tanhf(x); }); break;
          case VM_ERF: top = map4(a, [](float x) { return erff(x); }); break;
          case VM_SIN: top = map4(a, [](float x) { return sinf(x); }); break;
          case VM_COS: top = map4(a, [](float x) { return cosf(x); }); break;
          case VM_ABS: top = map4(a, [](float x) { return fabsf(x); }); break;
          case VM_FLOOR: top = map4(a, [](float x) { return floorf(x); }); break;
          case VM_CEIL: top = map4(a, [](float x) { return ceilf(x); }); break;
          default: top = map4(a, [](float x) { return 1.0f / (1.0f + expf(-x)); }); break;  // VM_SIGMOID
        }
      }
    }
    const float4 r = top;
    if (vec) {
      if (p.out_f16) {
        uint2 h;
        h.x = h22u(__floats2half2_rn(r.x, r.y));
        h.y = h22u(__floats2half2_rn(r.z, r.w));
        *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.out) + i) = h;
      } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + i) = r;
      }
    } else {
      const float e[4] = {r.x, r.y, r.z, r.w};
      for (int j = 0; j < 4; ++j)
        if (i + j < p.n) {
          if (p.out_f16) reinterpret_cast<__half *>(p.out)[i + j] = __float2half_rn(e[j]);
          else reinterpret_cast<float *>(p.out)[i + j] = e[j];
        }
    }
  }
}

}  // namespace ab200

using namespace ab200;

// ops / args: the stack program (n_ops entries, codes as in VmOp); consts: fp32 constants; inputs:
// device pointers with their dtypes (AB200_F16 / AB200_F32); every input and the output hold n elements.
extern "C" int ab200_eltwise_vm(const unsigned char *ops_host, const unsigned char *args_host, int n_ops, const float *consts_host, int n_consts,
                                const void *const *inputs_host, const int *in_dtypes_host, int n_inputs, void *out, int out_dtype, size_t n,
                                void *stream) {
  clear_error();
  AB200_REQUIRE(ops_host && args_host && inputs_host && in_dtypes_host && out, "eltwise_vm: null pointer");
  AB200_REQUIRE(n_ops >= 1 && n_ops <= VM_MAX_OPS && n_consts >= 0 && n_consts <= VM_MAX_CONSTS && n_inputs >= 1 && n_inputs <= VM_MAX_INPUTS,
                "eltwise_vm: program of %d ops, %d constants, %d inputs exceeds the interpreter (max %d / %d / %d)", n_ops, n_consts, n_inputs,
                VM_MAX_OPS, VM_MAX_CONSTS, VM_MAX_INPUTS);
  AB200_REQUIRE(n_consts == 0 || consts_host != nullptr, "eltwise_vm: constants missing");
  if (n == 0) return AB200_OK;
  VmProgram p{};
  int depth = 0, vec_ok = 1;
  for (int k = 0; k < n_ops; ++k) {  // validate on the host: the kernel trusts the program
    const int op = ops_host[k], arg = args_host[k];
    AB200_REQUIRE(op < VM_OP_COUNT, "eltwise_vm: unknown operation code %d", op);
    if (op == VM_IN) {
      AB200_REQUIRE(arg < n_inputs, "eltwise_vm: input index %d out of range", arg);
      ++depth;
    } else if (op == VM_CONST) {
      AB200_REQUIRE(arg < n_consts, "eltwise_vm: constant index %d out of range", arg);
      ++depth;
    } else if (op <= VM_DIV || (op >= VM_MAX && op <= VM_POW)) {
      AB200_REQUIRE(depth >= 2, "eltwise_vm: stack underflow at operation %d", k);
      --depth;
    } else {
      AB200_REQUIRE(depth >= 1, "eltwise_vm: stack underflow at operation %d", k);
    }
    AB200_REQUIRE(depth <= VM_MAX_STACK, "eltwise_vm: expression needs more than %d stack slots", VM_MAX_STACK);
    p.op[k] = (unsigned char)op;
    p.arg[k] = (unsigned char)arg;
  }
  AB200_REQUIRE(depth == 1, "eltwise_vm: the program leaves %d values on the stack", depth);
  for (int j = 0; j < n_consts; ++j) p.cst[j] = consts_host[j];
  for (int j = 0; j < n_inputs; ++j) {
    AB200_REQUIRE(inputs_host[j] != nullptr && (in_dtypes_host[j] == AB200_F16 || in_dtypes_host[j] == AB200_F32), "eltwise_vm: bad input %d", j);
    p.in[j] = inputs_host[j];
    p.in_f16[j] = in_dtypes_host[j] == AB200_F16;
    if (!aligned16(inputs_host[j])) vec_ok = 0;
  }
  AB200_REQUIRE(out_dtype == AB200_F16 || out_dtype == AB200_F32, "eltwise_vm: bad output dtype %d", out_dtype);
  if (!aligned16(out)) vec_ok = 0;
  p.out = out;
  p.out_f16 = out_dtype == AB200_F16;
  p.n_ops = n_ops;
  p.n = n;
  const size_t n4 = (n + 3) / 4;
  size_t blocks = (n4 + VM_THREADS - 1) / VM_THREADS;
  const size_t cap = (size_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  eltwise_vm_kernel<<<(unsigned)blocks, VM_THREADS, 0, (cudaStream_t)stream>>>(p, vec_ok);
  AB200_CHECK_LAUNCH("eltwise_vm");
  return AB200_OK;
}

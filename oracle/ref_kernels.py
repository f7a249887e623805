"""Kernel-source texts for the reference's c-mcpu runtime (TEST INFRASTRUCTURE ONLY).

The reference turns Antares IR into kernel source through a patched TVM that cannot be installed
offline, so each IR statement on the hot path is restated here by hand as the loop nest the IR
defines (AntaresIR.md:33-49), in the wire format and C dialect the reference produces:

  header   `// GLOBALS: a:dtype[d0, d1], ... -> out:dtype[...]`, `// BACKEND: c-mcpu (default)`
           (antares/antares_compiler.py:183-199; parsed graph_evaluator/execute_module.hpp:277-283)
  slices   separated by a dashed line, each `// LOCAL: name -- ins -> outs` with a
           `// [thread_extent] __rank__ = R` line (execute_module.hpp:285-318)
  body     `extern "C" void f(const int __rank__, void** __args)` with `half` spelled `__fp16`
           (backends/c-scpu/config.py:22-49).  x86 g++ has no `__fp16`; `_Float16` is the same
           IEEE binary16 type, hence the #define at the top of each fp16 source.
  split    reduce ops: __rank__ = tiles of 64 outputs, inner order [2][K/4][8][4][4]
           (backends/c-mcpu/schedule/standard/default.py:11-46); elementwise ops: one output
           element per __rank__ (default.py:48-56).

The texts are compiled by the reference's own, unmodified `ab::moduleCompile`
(g++ -O2 -ffast-math, backends/c-mcpu/include/backend.hpp:148-164).
"""

SEP = "// ---------------------------------------------------------------------------\n"

_PRELUDE = """
#include <math.h>
#include <algorithm>
#define rsqrt(x)  (1.0f / sqrt(x))
#define __fp16 _Float16
"""

_CT = {"float16": "__fp16", "float32": "float", "int32": "int"}


def _sig(tensors):
    return ", ".join("%s:%s[%s]" % (n, d, ", ".join(str(int(x)) for x in s)) for n, d, s in tensors)


def _args(ins, outs):
    lines = []
    for i, (n, d, _) in enumerate(ins):
        lines.append("  auto* %s = (%s* __restrict)__args[%d];" % (n, _CT[d], i))
    for i, (n, d, _) in enumerate(outs):
        lines.append("  auto* %s = (%s*)__args[%d];" % (n, _CT[d], i + len(ins)))
    return "\n".join(lines)


def _kernel(name, ins, outs, rank_extent, body):
    return (SEP + "// LOCAL: %s -- %s -> %s\n" % (name, _sig(ins), _sig(outs)) + _PRELUDE +
            '\nextern "C" void %s(const int __rank__, void** __args) {\n%s\n  using namespace std;\n'
            "  // [thread_extent] __rank__ = %d\n%s\n}\n" % (name, _args(ins, outs), rank_extent, body))


def _module(ins, outs, compute_v1, kernels):
    head = ("// GLOBALS: %s -> %s\n// BACKEND: c-mcpu (default)\n// CONFIG: null\n// COMPUTE_V1: %s\n\n"
            % (_sig(ins), _sig(outs), compute_v1.replace("\n", " ")))
    return head + "\n".join(kernels)


W4A16_IR = ("input1[S, N] = (qweight[S / 8, N] >> (S % 8 * 4)).call(strs.bitwise_and, 15) * input0[S].like(1); "
            "w[S, N] = scales[S / 128, N] * (input1[S, N] - 8); "
            "my_result[N] +=! input0[S] * w[S, N].to(input0.dtype())")


def w4a16(M, K, N, dtype="float16", group=128):
    """The three statements of samples/05_llama2_7b_int4.py:135-139, inlined into one reduce
    kernel (the reference inlines every non-reduce stage, antares/default_codegen.py:239-258).
    fp32 accumulator; w rounded to the scales' dtype as statement 2 declares."""
    assert N % 64 == 0 and K % 8 == 0 and K % group == 0
    ins = [("input0", dtype, (M, K)), ("qweight", "int32", (K // 8, N)), ("scales", dtype, (K // group, N))]
    outs = [("my_result", dtype, (M, N))]
    t = _CT[dtype]
    body = """
  const int K = %d, N = %d, M = %d, G = %d;
  const int n_base = __rank__ * 64;
  for (int m = 0; m < M; ++m) {
    float acc[64];
    for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
    for (int n1 = 0; n1 < 2; ++n1)
      for (int ko = 0; ko < K / 4; ++ko)
        for (int n2 = 0; n2 < 8; ++n2)
          for (int ki = 0; ki < 4; ++ki)
            for (int n3 = 0; n3 < 4; ++n3) {
              const int S = ko * 4 + ki, c = n1 * 32 + n2 * 4 + n3, n = n_base + c;
              %s input1 = (%s)((qweight[(S / 8) * N + n] >> (S %% 8 * 4)) & 15);
              %s w = scales[(S / G) * N + n] * (input1 - (%s)8);
              acc[c] += (float)input0[m * K + S] * (float)w;
            }
    for (int i = 0; i < 64; ++i) my_result[m * N + n_base + i] = (%s)acc[i];
  }""" % (K, N, M, group, t, t, t, t, t)
    return _module(ins, outs, W4A16_IR, [_kernel("template_op_kernel0", ins, outs, N // 64, body)])


def w4_dequant(K, N, dtype="float16", group=128):
    """Statements 1-2 alone with `w` as the output: the dequantised weight that must be bit-exact."""
    ins = [("qweight", "int32", (K // 8, N)), ("scales", dtype, (K // group, N))]
    outs = [("w", dtype, (K, N))]
    t = _CT[dtype]
    body = """
  const int N = %d, G = %d, S = __rank__;
  for (int n = 0; n < N; ++n) {
    %s input1 = (%s)((qweight[(S / 8) * N + n] >> (S %% 8 * 4)) & 15);
    w[S * N + n] = scales[(S / G) * N + n] * (input1 - (%s)8);
  }""" % (N, group, t, t, t)
    ir = "input1[S, N] = ...; w[S, N] = scales[S / 128, N] * (input1[S, N] - 8)"
    return _module(ins, outs, ir, [_kernel("template_op_kernel0", ins, outs, K, body)])


def sigmoid_f32(N):
    """README.md:66: sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp)).  Elementwise default
    schedule = one element per rank; ranks are grouped by 1024 here so that the rank count stays
    within int range for large N and the pool's per-rank call does not dominate."""
    ins, outs = [("data", "float32", (N,))], [("sigmoid_f32", "float32", (N,))]
    ranks = (N + 1023) // 1024
    body = """
  for (int i = __rank__ * 1024; i < %d && i < (__rank__ + 1) * 1024; ++i)
    sigmoid_f32[i] = 1.0f - 1.0f / (1.0f + expf(data[i]));""" % N
    return _module(ins, outs, "sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp))",
                   [_kernel("template_op_kernel0", ins, outs, ranks, body)])


def softmax(rows, cols, dtype="float16"):
    """AntaresIR.md:226, three statements -> three chained kernels with two temporaries, which
    exercises ExecutionModule's intermediate allocation (execute_module.hpp:336-358)."""
    t = _CT[dtype]
    x = ("input0", dtype, (rows, cols))
    t0, t1 = ("temp0", "float32", (rows,)), ("temp1", "float32", (rows,))
    o = ("output0", dtype, (rows, cols))
    k0 = _kernel("template_op_kernel0", [x], [t0], rows, """
  float m = -INFINITY;
  for (int c = 0; c < %d; ++c) m = max(m, (float)input0[__rank__ * %d + c]);
  temp0[__rank__] = m;""" % (cols, cols))
    k1 = _kernel("template_op_kernel1", [x, t0], [t1], rows, """
  float s = 0.0f;
  for (int c = 0; c < %d; ++c) s += expf((float)input0[__rank__ * %d + c] - temp0[__rank__]);
  temp1[__rank__] = s;""" % (cols, cols))
    k2 = _kernel("template_op_kernel2", [x, t0, t1], [o], rows, """
  for (int c = 0; c < %d; ++c)
    output0[__rank__ * %d + c] = (%s)(expf((float)input0[__rank__ * %d + c] - temp0[__rank__]) / temp1[__rank__]);"""
                 % (cols, cols, t, cols))
    ir = ("temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); "
          "output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]")
    return _module([x], [o], ir, [k0, k1, k2])


def rmsnorm_vsum_f32(N, eps=1e-6):
    """Signature of autort.ops.rmsnorm_f32 (samples/05_llama2_7b_int4.py:128-131); the IR is in a
    closed wheel, so the body is the standard Llama-2 RMSNorm (parity unpinned).  The scalar
    `extra=[1/N]` becomes a compile-time constant."""
    ins = [("vsum", "float32", (1,)), ("weight", "float32", (N,)), ("x", "float32", (N,))]
    outs = [("rmsnorm_f32", "float32", (N,))]
    ranks = (N + 63) // 64
    body = """
  const float rs = 1.0f / sqrtf(vsum[0] * %.10ef + %.10ef);
  for (int i = __rank__ * 64; i < %d && i < (__rank__ + 1) * 64; ++i)
    rmsnorm_f32[i] = x[i] * rs * weight[i];""" % (1.0 / N, eps, N)
    return _module(ins, outs, "rmsnorm_f32[N] = x[N] * (vsum[0] * inv_n + eps).call(`rsqrt`) * weight[N]",
                   [_kernel("template_op_kernel0", ins, outs, ranks, body)])


def rmsnorm_rows(rows, cols, dtype="float16", eps=1e-6):
    """Row-wise RMSNorm over [rows, cols] (sum of squares + scale in one op)."""
    t = _CT[dtype]
    ins = [("weight", dtype, (cols,)), ("x", dtype, (rows, cols))]
    outs = [("rmsnorm", dtype, (rows, cols))]
    body = """
  const int C = %d;
  float vsum = 0.0f;
  for (int c = 0; c < C; ++c) vsum += (float)x[__rank__ * C + c] * (float)x[__rank__ * C + c];
  const float rs = 1.0f / sqrtf(vsum * (1.0f / C) + %.10ef);
  for (int c = 0; c < C; ++c)
    rmsnorm[__rank__ * C + c] = (%s)((float)x[__rank__ * C + c] * rs * (float)weight[c]);""" % (cols, eps, t)
    return _module(ins, outs, "rmsnorm rows", [_kernel("template_op_kernel0", ins, outs, rows, body)])


def rotary(rows, H, D, dtype="float16"):
    """Signature of autort.ops.rotary_f32(x[H,2,D/2], inv_freq[D], out[H,D], extra=[pos])
    (samples/05_llama2_7b_int4.py:157-158), batched over rows with a position per row; body is
    the rotate-half definition (closed op, parity unpinned)."""
    t = _CT[dtype]
    ins = [("inv_freq", "float32", (D,)), ("pos", "int32", (rows,)), ("x", dtype, (rows, H, D))]
    outs = [("rotary", dtype, (rows, H, D))]
    body = """
  const int H = %d, D = %d, r = __rank__ / H;
  const %s* xi = x + (long)__rank__ * D;
  %s* oi = rotary + (long)__rank__ * D;
  for (int j = 0; j < D / 2; ++j) {
    float th = (float)pos[r] * inv_freq[j];
    float c = cosf(th), s = sinf(th);
    float a = (float)xi[j], b = (float)xi[j + D / 2];
    oi[j] = (%s)(a * c - b * s);
    oi[j + D / 2] = (%s)(b * c + a * s);
  }""" % (H, D, t, t, t, t)
    return _module(ins, outs, "rotary rotate-half", [_kernel("template_op_kernel0", ins, outs, rows * H, body)])


def attention(S, H, D, kv_rows, dtype="float16", scale=None):
    """Signature of autort.ops.attention_f32(q[H,D], K[S,H,D], V[S,H,D], att_f[1])
    (samples/05_llama2_7b_int4.py:161-165); caches are declared with `kv_rows` rows and the first
    S are used.  Body = single-query softmax attention (closed op, parity unpinned)."""
    t = _CT[dtype]
    ins = [("att_f", "float32", (1,)), ("k", dtype, (kv_rows, H, D)), ("q", dtype, (H, D)), ("v", dtype, (kv_rows, H, D))]
    outs = [("attention", dtype, (H, D))]
    body = """
  const int S = %d, H = %d, D = %d, h = __rank__;
  float p[%d];
  float mx = -INFINITY, sum = 0.0f;
  for (int s = 0; s < S; ++s) {
    float dot = 0.0f;
    for (int d = 0; d < D; ++d) dot += (float)q[h * D + d] * (float)k[((long)s * H + h) * D + d];
    p[s] = dot * att_f[0];
    mx = max(mx, p[s]);
  }
  for (int s = 0; s < S; ++s) { p[s] = expf(p[s] - mx); sum += p[s]; }
  for (int d = 0; d < D; ++d) {
    float acc = 0.0f;
    for (int s = 0; s < S; ++s) acc += p[s] * (float)v[((long)s * H + h) * D + d];
    attention[h * D + d] = (%s)(acc / sum);
  }""" % (S, H, D, S, t)
    return _module(ins, outs, "single-query attention", [_kernel("template_op_kernel0", ins, outs, H, body)])

"""GPU tests of the drop-in surface: the call sites of the reference's samples, verbatim, against the
CPU oracle.  Tolerance: max|err| <= 1e-2 * max|ref| (fp32 variants much tighter)."""
import math

import numpy as np
import pytest
import torch

import autort
from antares_b200 import packing
from antares_b200.custom_op import CustomOp
from oracle import cport

pytestmark = pytest.mark.gpu

W4A16_IR = """
  input1[S, N] = (qweight[S / 8, N] >> (S % 8 * 4)).call(strs.bitwise_and, 15) * input0[S].like(1)
  w[S, N] = scales[S / 128, N] * (input1[S, N] - 8)
  my_result[N] +=! input0[S] * w[S, N].to(input0.dtype())
"""


def _err(y, ref):
    y, ref = np.asarray(y, np.float32), np.asarray(ref, np.float32)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


def test_export_w4a16_as_in_the_int4_sample(cuda):
    """samples/05_llama2_7b_int4.py:135-144 with its own dtypes (fp32 x and scales), out= and dynamic dims."""
    fn = autort.export(ir=W4A16_IR, inputs=["input0=float32[S:4096]", "qweight=int32[L:512, N:12288]", "scales=float32[K:32, N:12288]"],
                       config="~N~:[256,8,32],~S~:[64,8]")
    assert autort.ops.my_result is fn
    for N in (12288, 4096):  # one exported op serves every projection (dims are upper bounds)
        qw, sc = packing.synth_w4(4096, N, 3, scales_dtype=np.float32)
        x = packing.synth_x(1, 4096, 4, np.float32)[0]
        ref = cport.w4a16_gemm(x, qw, sc)
        dev = autort.device()
        out = torch.empty(N, dtype=torch.float32, device=dev)
        res = fn(torch.from_numpy(x).to(dev), torch.from_numpy(qw).to(dev), torch.from_numpy(sc).to(dev), out=out.view(-1))
        assert res.data_ptr() == out.data_ptr()
        assert _err(out.cpu().numpy(), ref) <= 1e-4
    with pytest.raises(ValueError):
        fn(torch.zeros(8192, device=dev), torch.zeros(1024, 64, dtype=torch.int32, device=dev), torch.zeros(64, 64, device=dev))


def test_export_sigmoid_as_in_the_readme(cuda):
    data = torch.arange(0, 10, dtype=torch.float32, device=autort.device())
    f = autort.export(ir="sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp))", inputs=["data=float32[N:4096000]"], config="tune:5")
    want = [0.5000, 0.7311, 0.8808, 0.9526, 0.9820, 0.9933, 0.9975, 0.9991, 0.9997, 0.9999]  # README.md:67
    assert np.allclose(f(data).cpu().numpy(), want, atol=1e-4)
    assert np.allclose(autort.ops.sigmoid_f32(data).cpu().numpy(), want, atol=1e-4)


def test_builtin_llama_ops_follow_the_sample_call_sites(cuda):
    dev = autort.device()
    rng = np.random.default_rng(0)
    n_heads, head_size, dim, pos = 32, 128, 4096, 5
    # rmsnorm (samples/05_llama2_7b_int4.py:128-131)
    x = torch.from_numpy(rng.standard_normal(dim).astype(np.float32)).to(dev)
    wgt = torch.from_numpy((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)).to(dev)
    vsum = (x * x).sum().view(1)
    y = autort.ops.rmsnorm_f32(x.view(-1), vsum, wgt, extra=[1.0 / int(x.numel())])
    ref = cport.rmsnorm_vsum_f32(x.cpu().numpy(), vsum.cpu().numpy(), wgt.cpu().numpy(), 1.0 / dim)
    assert _err(y.cpu().numpy(), ref) <= 1e-5
    # rotary (lines 125-126, 157-158)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_size, 2).float() / head_size)))
    inv_freq = torch.cat([inv_freq, inv_freq]).view(head_size).to(dev)
    sq = torch.from_numpy(rng.standard_normal(dim).astype(np.float32)).to(dev)
    sq_out = torch.empty_like(sq).view(n_heads, head_size)
    autort.ops.rotary_f32(sq.view(n_heads, 2, -1), inv_freq, sq_out, extra=[pos, ])
    ref = cport.rope(sq.cpu().numpy().astype(np.float16).reshape(1, n_heads, head_size), np.array([pos], np.int32), inv_freq.cpu().numpy())
    assert _err(sq_out.cpu().numpy(), ref[0]) <= 2e-3
    # attention (lines 161-165): caches narrowed to pos + 1 rows
    kc = torch.from_numpy(rng.standard_normal((256, dim)).astype(np.float16)).to(dev)
    vc = torch.from_numpy(rng.standard_normal((256, dim)).astype(np.float16)).to(dev)
    q = torch.from_numpy(rng.standard_normal((n_heads, head_size)).astype(np.float16)).to(dev)
    att_f = torch.tensor([1 / math.sqrt(head_size)], dtype=torch.float32, device=dev)
    b_sk = kc.view(256, n_heads, head_size).narrow(0, 0, pos + 1)
    b_sv = vc.view(256, n_heads, head_size).narrow(0, 0, pos + 1)
    xb = autort.ops.attention_f16(q, b_sk, b_sv, att_f)
    ref = cport.attention_decode(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), pos + 1, 1 / math.sqrt(head_size))
    assert _err(xb.cpu().numpy(), ref) <= 1e-2
    xb32 = autort.ops.attention_f32(q.float(), b_sk.float(), b_sv.float(), att_f)
    assert _err(xb32.cpu().numpy(), ref) <= 2e-3


def test_legacy_custom_op_binding(cuda):
    """frameworks/pytorch/custom_op.py protocol: CustomOp(ir, input_orders, device).tune().emit(); op(*inputs)."""
    dev = autort.device()
    qw, sc = packing.synth_w4(512, 256, 9)
    x = packing.synth_x(1, 512, 10)[0]
    t = dict(input0=torch.from_numpy(x).to(dev), qweight=torch.from_numpy(qw).to(dev), scales=torch.from_numpy(sc).to(dev))
    op = CustomOp(ir=W4A16_IR, input_orders=t, device=dev).tune(step=0).emit()
    y = op(t["input0"], t["qweight"], t["scales"])
    assert _err(y.cpu().numpy(), cport.w4a16_gemm(x, qw, sc)) <= 1e-2
    sm = CustomOp(ir="temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); "
                     "output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]",
                  input_orders={"input0": (None, torch.float32, [32, 1024])}, device=dev).emit()
    xs = torch.randn(32, 1024, device=dev)
    assert torch.allclose(sm(xs), torch.softmax(xs, -1), atol=1e-6)
    add = CustomOp(ir="output0[N] = input0[N] + input1[N]", input_orders={"input0": xs[0], "input1": xs[1]}, device=dev).emit()
    assert torch.equal(add(xs[0], xs[1]), xs[0] + xs[1])       # a plain element-wise statement: the interpreter kernel
    with pytest.raises(NotImplementedError):                    # a dense matmul is outside the operator family
        CustomOp(ir="output0[N, M] +=! input0[N, K] * input1[K, M]", input_orders={"input0": xs, "input1": xs.t().contiguous()}, device=dev).emit()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("n", [4096 * 33, 1001])
def test_exported_elementwise_statements_run_on_the_interpreter(cuda, dtype, n):
    """autort.export of single element-wise statements outside the named family (the reference
    compiles a kernel per statement): tanh-GELU, a fused scaled residual, and a two-input
    expression with max/abs/rsqrt, against numpy in fp32."""
    import autort
    from antares_b200 import ir
    dt = "float32" if dtype == torch.float32 else "float16"
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    y = (rng.standard_normal(n) * 2).astype(np.float32)
    xd, yd = torch.from_numpy(x).to(cuda).to(dtype), torch.from_numpy(y).to(cuda).to(dtype)
    xr, yr = xd.float().cpu().numpy(), yd.float().cpu().numpy()
    tol = 1e-5 if dtype == torch.float32 else 2e-3
    gelu = autort.export(ir="out[N] = 0.5 * x[N] * (1.0 + (0.7978845608 * (x[N] + 0.044715 * x[N] * x[N] * x[N])).call(`tanh`))",
                         inputs=["x=%s[N:%d]" % (dt, 1 << 22)], name="gelu_tanh")
    assert gelu.match.kind == "eltwise"
    got = autort.ops.gelu_tanh(xd).float().cpu().numpy()
    want = 0.5 * xr * (1 + np.tanh(0.7978845608 * (xr + 0.044715 * xr ** 3)))
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())
    fused = autort.export(ir="z[N] = a[N] + 0.125 * (b[N] - a[N]).call(strs.max, [const(0.0)]) * (b[N].call(`abs`) + 1.0).call(`rsqrt`)",
                          inputs=["a=%s[N:%d]" % (dt, 1 << 22), "b=%s[N:%d]" % (dt, 1 << 22)])
    out = torch.empty(n, dtype=dtype, device=cuda)
    fused(xd, yd, out)                       # trailing output tensor, as samples/05_llama2_7b_int4.py:157 passes it
    want = xr + 0.125 * np.maximum(yr - xr, 0) / np.sqrt(np.abs(yr) + 1)
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
    # an odd offset view (not 16-byte aligned) takes the scalar path
    if n > 8:
        got = autort.ops.gelu_tanh(xd[1:]).float().cpu().numpy()
        want = 0.5 * xr[1:] * (1 + np.tanh(0.7978845608 * (xr[1:] + 0.044715 * xr[1:] ** 3)))
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


def test_native_inject_forward_against_oracle(cuda):
    """Kernel-source text in the reference's wire format -> ab200_inject -> key -> ab200_forward with raw
    pointers (inputs sorted by name, then the output): W4A16, sigmoid and row softmax against the oracle."""
    import ctypes
    from antares_b200 import ops
    from antares_b200._lib import call
    st = torch.cuda.current_stream().cuda_stream

    def inject(globals_line, ir):
        text = ("// GLOBALS: %s\n// BACKEND: c-b200 (default)\n// CONFIG: \n// COMPUTE_V1: - einstein_v2(input_dict={}, extra_outputs=[], exprss=\"%s\")\n"
                % (globals_line, ir))
        key = ctypes.c_int(-1)
        call("ab200_inject", text.encode(), ctypes.cast(ctypes.pointer(key), ctypes.c_void_p))
        return key.value

    def forward(key, *tensors):
        args = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        call("ab200_forward", key, ctypes.cast(args, ctypes.c_void_p), len(tensors), st)

    K, N = 4096, 4096
    qw, sc = packing.synth_w4(K, N, 0)
    x = packing.synth_x(1, K, 1)
    ir = "; ".join(s.strip() for s in W4A16_IR.strip().split("\n"))
    key = inject("input0:float16[%d], qweight:int32[%d, %d], scales:float16[%d, %d] -> my_result:float16[%d]" % (K, K // 8, N, K // 128, N, N), ir)
    y = torch.empty(N, dtype=torch.float16, device=cuda)
    forward(key, torch.from_numpy(x[0]).to(cuda), torch.from_numpy(qw).to(cuda), torch.from_numpy(sc).to(cuda), y)
    assert _err(y.cpu().numpy(), cport.w4a16_gemm(x, qw, sc)[0]) <= 1e-2
    # 32 rows: the same text family is served by the tensor-core kernel
    x32 = packing.synth_x(128, K, 2)
    key = inject("input0:float16[128, %d], qweight:int32[%d, %d], scales:float16[%d, %d] -> my_result:float16[128, %d]" % (K, K // 8, N, K // 128, N, N), ir)
    y2 = torch.empty((128, N), dtype=torch.float16, device=cuda)
    forward(key, torch.from_numpy(x32).to(cuda), torch.from_numpy(qw).to(cuda), torch.from_numpy(sc).to(cuda), y2)
    assert _err(y2.cpu().numpy(), cport.w4a16_gemm(x32, qw, sc)) <= 1e-2
    rng = np.random.default_rng(3)
    d = rng.standard_normal(5000).astype(np.float32)
    key = inject("data:float32[5000] -> sigmoid_f32:float32[5000]", "sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp))")
    o = torch.empty(5000, dtype=torch.float32, device=cuda)
    forward(key, torch.from_numpy(d).to(cuda), o)
    assert np.abs(o.cpu().numpy() - cport.sigmoid(d)).max() <= 1e-6
    s_in = (3 * rng.standard_normal((32, 4096))).astype(np.float16)
    key = inject("input0:float16[32, 4096] -> output0:float16[32, 4096]",
                 "temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]")
    so = torch.empty((32, 4096), dtype=torch.float16, device=cuda)
    forward(key, torch.from_numpy(s_in).to(cuda), so)
    assert _err(so.cpu().numpy(), cport.softmax(s_in)) <= 1e-2
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0


def test_layernorm_ir_runs_on_the_row_reduction_template(cuda):
    """The layernorm program of AntaresIR.md:232 through autort.export (three statements: two row sums and
    a map), fp32 and fp16, against numpy; and a variant with per-column weight and bias through CustomOp."""
    ln = ("temp0[N] +=! input0[N, C]; temp1[N] +=! input0[N, C] * input0[N, C]; "
          "output0[N, C] = (input0[N, C] * C.val() - temp0[N]) * (temp1[N] * C.val() - temp0[N] * temp0[N] + 1e-5).call(`rsqrt`)")
    f = autort.export(ir=ln, inputs=["input0=float32[N:32, C:1024]"], name="layernorm_f32")
    x = np.random.default_rng(0).standard_normal((32, 1024)).astype(np.float32) * 2 + 0.5
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5 / 1024 ** 2)
    y = autort.ops.layernorm_f32(torch.from_numpy(x).to(cuda))
    assert y.dtype == torch.float32 and np.abs(y.cpu().numpy() - want).max() <= 5e-4
    y2 = f(torch.from_numpy(x[:7]).to(cuda))        # fewer rows than declared: N is a dynamic axis
    assert np.abs(y2.cpu().numpy() - want[:7]).max() <= 5e-4
    ir2 = ("s[N] +=! x[N, C]; q[N] +=! x[N, C] * x[N, C]; "
           "y[N, C] = (x[N, C] - s[N] / C.val()) * (q[N] / C.val() - s[N] / C.val() * s[N] / C.val() + 1e-5).call(`rsqrt`) * g[C] + b[C]")
    xh = np.random.default_rng(1).standard_normal((2048, 4096)).astype(np.float16)
    g = np.linspace(0.5, 1.5, 4096).astype(np.float16)
    b = np.linspace(-1, 1, 4096).astype(np.float16)
    op = CustomOp(ir=ir2, input_orders={"x": torch.from_numpy(xh), "g": torch.from_numpy(g), "b": torch.from_numpy(b)}, device=cuda).emit()
    yh = op(torch.from_numpy(xh), torch.from_numpy(g), torch.from_numpy(b))
    xf = xh.astype(np.float32)
    want2 = (xf - xf.mean(-1, keepdims=True)) / np.sqrt(xf.var(-1, keepdims=True) + 1e-5) * g.astype(np.float32) + b.astype(np.float32)
    assert yh.dtype == torch.float16 and _err(yh.cpu().numpy(), want2) <= 1e-2
    # bitwise repeatable (fixed reduction order)
    assert torch.equal(op(torch.from_numpy(xh), torch.from_numpy(g), torch.from_numpy(b)), yh)

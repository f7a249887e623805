"""CPU tests of the IR recogniser and the AutoRT-style declarations (no kernel is launched)."""
import pytest

from antares_b200 import ir
from vm_ref import eval_program_numpy

W4A16_IR = """
  input1[S, N] = (qweight[S / 8, N] >> (S % 8 * 4)).call(strs.bitwise_and, 15) * input0[S].like(1)
  w[S, N] = scales[S / 128, N] * (input1[S, N] - 8)
  my_result[N] +=! input0[S] * w[S, N].to(input0.dtype())
"""
W4A16_INPUTS = ["input0=float32[S:4096]", "qweight=int32[L:512, N:12288]", "scales=float32[K:32, N:12288]"]


def test_input_spec_parsing():
    s = ir.parse_input_spec("qweight=int32[L:512, N:12288]")
    assert (s.name, s.dtype, s.dims, s.dyn) == ("qweight", "int32", [512, 12288], ["L", "N"])
    s = ir.parse_input_spec("data=float32[N:4096000]")
    assert s.dims == [4096000] and s.dyn == ["N"]
    s = ir.parse_input_spec("x=float16[32, 1024]")
    assert s.dyn == [None, None]
    with pytest.raises(ValueError):
        ir.parse_input_spec("x=float7[3]")


def test_recognises_the_sample_w4a16_program():
    m = ir.recognise(W4A16_IR, W4A16_INPUTS)
    assert m.kind == "w4a16" and m.name == "my_result"          # default name = last l-value (README.md:66-69)
    assert m.params == dict(x="input0", qweight="qweight", scales="scales", group=128, dtype="float32")
    m = ir.recognise(W4A16_IR.replace("\n", " ; ").replace("+=!", "+="), [t.replace("float32", "float16") for t in W4A16_INPUTS], name="q4")
    assert m.name == "q4" and m.params["dtype"] == "float16"
    m = ir.recognise(W4A16_IR.replace("/ 128", "/ 64"), W4A16_INPUTS)
    assert m.params["group"] == 64


def test_recognises_sigmoid_and_softmax():
    m = ir.recognise("sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp))", ["data=float32[N:4096000]"])
    assert m.kind == "sigmoid" and m.name == "sigmoid_f32"
    m = ir.recognise("output0[N, M] = 1.0 / (1.0 + (-input0[N, M]).call(`exp`))", ["input0=float32[1024, 512]"])
    assert m.kind == "sigmoid"
    sm = ("temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); "
          "output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]")
    m = ir.recognise(sm, ["input0=float16[32, 4096]"])
    assert m.kind == "softmax" and m.output == "output0"


def test_everything_else_is_refused_not_emulated():
    with pytest.raises(NotImplementedError):   # a matmul: neither W4A16 nor element-wise
        ir.recognise("output0[N, M] +=! input0[N, K] * input1[K, M]", ["input0=float32[8, 8]", "input1=float32[8, 8]"])
    with pytest.raises(NotImplementedError):   # integer element-wise (the interpreter computes in fp32)
        ir.recognise("output0[N] = input0[N] + input1[N]", ["input0=int32[8]", "input1=int32[8]"])
    with pytest.raises(NotImplementedError):   # zero-point other than 8
        ir.recognise(W4A16_IR.replace("- 8)", "- 7)"), W4A16_INPUTS)
    with pytest.raises(NotImplementedError):   # mixed dtypes
        ir.recognise(W4A16_IR, ["input0=float16[S:4096]", "qweight=int32[L:512, N:12288]", "scales=float32[K:32, N:12288]"])


def test_elementwise_statements_compile_to_stack_programs():
    """Single element-wise statements outside the named family go to the interpreter: the stack
    program evaluates to the expression (numpy), constants are pooled, casts are no-ops."""
    import numpy as np
    from antares_b200 import ir
    gelu = "out[N] = 0.5 * x[N] * (1.0 + (0.7978845608 * (x[N] + 0.044715 * x[N] * x[N] * x[N])).call(`tanh`))"
    m = ir.recognise(gelu, ["x=float32[N:4096]"])
    assert m.kind == "eltwise" and m.name == "out" and m.params["inputs"] == ["x"]
    x = np.linspace(-4, 4, 33).astype(np.float32)
    got = eval_program_numpy(m.params["program"], m.params["consts"], [x])
    assert np.allclose(got, 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3))), atol=1e-6)
    m = ir.recognise("y[A, B] = (a[A, B] - b[A, B]).call(strs.max, [const(0.0)]) / -c[A, B].cast(`float32`) + a[A, B]",
                     ["a=float16[8, 16]", "b=float16[8, 16]", "c=float32[8, 16]"], name="fused")
    assert m.kind == "eltwise" and m.name == "fused" and m.params["inputs"] == ["a", "b", "c"] and m.params["axes"] == ["A", "B"]
    rng = np.random.default_rng(0)
    a, b, c = (rng.standard_normal((8, 16)).astype(np.float32) for _ in range(3))
    got = eval_program_numpy(m.params["program"], m.params["consts"], [a, b, c])
    assert np.allclose(got, np.maximum(a - b, 0) / -c + a, rtol=1e-6)


@pytest.mark.parametrize("bad", ["out[N] = x[N + 1] * 2.0",                 # shifted index: not element-wise
                                 "out[N] = x[N].call(`frobnicate`)",        # unknown function
                                 "out[N] +=! x[N, M]",                      # a reduction
                                 "out[N] = 1.0"])                           # reads nothing
def test_non_elementwise_statements_are_refused(bad):
    from antares_b200 import ir
    with pytest.raises(NotImplementedError):
        ir.recognise(bad, ["x=float32[N:64]"])


LAYERNORM_IR = ("temp0[N] +=! input0[N, C]; temp1[N] +=! input0[N, C] * input0[N, C]; "
                "output0[N, C] = (input0[N, C] * C.val() - temp0[N]) * (temp1[N] * C.val() - temp0[N] * temp0[N] + 1e-5).call(`rsqrt`)")
SOFTMAX_IR = ("temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); "
              "output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]")


def test_reduce_map_chains_compile_to_row_programs():
    """The layernorm program of AntaresIR.md:232 compiles to three stages (sum, sum, map) and evaluates to
    numpy's layernorm; a variant with a per-column weight and bias uses [C] operands."""
    import numpy as np
    from vm_ref import eval_row_program_numpy
    m = ir.recognise(LAYERNORM_IR, ["input0=float32[N:32, C:1024]"])
    assert m.kind == "rowprog" and m.output == "output0"
    rp = m.params
    assert [k for k, _ in rp["stages"]] == [1, 1, 0] and rp["mats"] == ["input0"] and rp["cols"] == []
    x = np.random.default_rng(0).standard_normal((32, 1024)).astype(np.float32) * 3 + 1
    got = eval_row_program_numpy(rp, [x], [])
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5 / 1024 ** 2)
    # the IR's form is (x C - sum) rsqrt(sumsq C - sum^2 + 1e-5): the same as (x - mean) / sqrt(var + 1e-5 / C^2)
    assert np.abs(got - want).max() <= 2e-4
    ir2 = ("s[N] +=! x[N, C]; q[N] +=! x[N, C] * x[N, C]; "
           "y[N, C] = (x[N, C] - s[N] / C.val()) * (q[N] / C.val() - s[N] / C.val() * s[N] / C.val() + 1e-5).call(`rsqrt`) * g[C] + b[C]")
    m2 = ir.recognise(ir2, ["x=float16[N:8, C:256]", "g=float16[C:256]", "b=float16[C:256]"], name="ln_affine")
    assert m2.kind == "rowprog" and m2.name == "ln_affine" and m2.params["cols"] == ["g", "b"]
    x2 = np.random.default_rng(1).standard_normal((8, 256)).astype(np.float32)
    g, b = np.linspace(0.5, 1.5, 256, dtype=np.float32), np.linspace(-1, 1, 256, dtype=np.float32)
    got2 = eval_row_program_numpy(m2.params, [x2], [g, b])
    want2 = (x2 - x2.mean(-1, keepdims=True)) / np.sqrt(x2.var(-1, keepdims=True) + 1e-5) * g + b
    assert np.abs(got2 - want2).max() <= 1e-4


def test_softmax_is_recognised_by_structure_not_by_text():
    """Whatever the tensors and axes are called, however the text is spaced, parenthesised or split into
    lines: a max / sum-of-exp / normalise chain is row softmax and gets the hand-written kernel."""
    for text, decl in ((SOFTMAX_IR, "input0=float16[N:32, C:4096]"),
                       ("m[R]>=!scores[R,K]\n z[R] += ((scores[R,K]) - m[R]).call(strs.exp)\n p[R,K] = ((scores[R,K] - m[R])).call(`exp`) / (z[R])", "scores=float32[R:4, K:100]")):
        m = ir.recognise(text, [decl])
        assert m.kind == "softmax" and m.params["x"] == decl.split("=")[0]
    # one change of substance and it is a generic row program again
    m = ir.recognise(SOFTMAX_IR.replace("/ temp1[N]", "/ (temp1[N] + 1.0)"), ["input0=float16[N:32, C:4096]"])
    assert m.kind == "rowprog"


def test_row_program_rejections():
    with pytest.raises(NotImplementedError):   # the reduced axis is not the last output axis
        ir.recognise("t[C] +=! x[N, C]; y[N, C] = x[N, C] - t[C]", ["x=float32[N:4, C:8]"])
    with pytest.raises(NotImplementedError):   # integer tensors
        ir.recognise("t[N] +=! x[N, C]; y[N, C] = x[N, C] - t[N]", ["x=int32[N:4, C:8]"])
    with pytest.raises(NotImplementedError):   # a reduction that is not closed by a map statement
        ir.recognise("t[N] +=! x[N, C]; u[N] +=! x[N, C] * t[N]", ["x=float32[N:4, C:8]"])

"""CPU tests of the IR recogniser and the AutoRT-style declarations (no kernel is launched)."""
import pytest

from antares_b200 import ir

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
    got = ir.eval_program_numpy(m.params["program"], m.params["consts"], [x])
    assert np.allclose(got, 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3))), atol=1e-6)
    m = ir.recognise("y[A, B] = (a[A, B] - b[A, B]).call(strs.max, [const(0.0)]) / -c[A, B].cast(`float32`) + a[A, B]",
                     ["a=float16[8, 16]", "b=float16[8, 16]", "c=float32[8, 16]"], name="fused")
    assert m.kind == "eltwise" and m.name == "fused" and m.params["inputs"] == ["a", "b", "c"] and m.params["axes"] == ["A", "B"]
    rng = np.random.default_rng(0)
    a, b, c = (rng.standard_normal((8, 16)).astype(np.float32) for _ in range(3))
    got = ir.eval_program_numpy(m.params["program"], m.params["consts"], [a, b, c])
    assert np.allclose(got, np.maximum(a - b, 0) / -c + a, rtol=1e-6)


@pytest.mark.parametrize("bad", ["out[N] = x[N + 1] * 2.0",                 # shifted index: not element-wise
                                 "out[N] = x[N].call(`frobnicate`)",        # unknown function
                                 "out[N] +=! x[N, M]",                      # a reduction
                                 "out[N] = 1.0"])                           # reads nothing
def test_non_elementwise_statements_are_refused(bad):
    from antares_b200 import ir
    with pytest.raises(NotImplementedError):
        ir.recognise(bad, ["x=float32[N:64]"])

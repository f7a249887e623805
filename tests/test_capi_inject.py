"""The native plugin boundary (ab200_inject / ab200_forward): header parsing and operator recognition
run on the host, so they are checked here without a GPU.  The wire format is the reference's
(antares/antares_compiler.py:183-199, graph_evaluator/execute_module.hpp:274-283)."""
import ctypes

import pytest

from antares_b200 import _lib

W4A16 = ('input1[S, N] = (qweight[S / 8, N] >> (S % 8 * 4)).call(strs.bitwise_and, 15) * input0[S].like(1); '
         'w[S, N] = scales[S / 128, N] * (input1[S, N] - 8); my_result[N] +=! input0[S] * w[S, N].to(input0.dtype())')


def _src(globals_line, ir, backend="c-b200"):
    return ("// GLOBALS: %s\n// BACKEND: %s (default)\n// CONFIG: \n// COMPUTE_V1: - einstein_v2(input_dict={}, extra_outputs=[], exprss=\"%s\")\n"
            "\n// ---------------------------------------------------------------------------\n// LOCAL: template_op_kernel0 -- x -> y\n" % (globals_line, backend, ir))


def _inject(text):
    L = _lib.load()
    key = ctypes.c_int(-1)
    rc = L.ab200_inject(text.encode(), ctypes.cast(ctypes.pointer(key), ctypes.c_void_p))
    return rc, key.value, L.ab200_last_error().decode()


def _tensor(key, slot):
    L = _lib.load()
    name, dtype = ctypes.create_string_buffer(64), ctypes.create_string_buffer(32)
    shape, rank = (ctypes.c_long * 8)(), ctypes.c_int(0)
    assert L.ab200_module_tensor(key, slot, ctypes.cast(name, ctypes.c_void_p), 64, ctypes.cast(dtype, ctypes.c_void_p), 32,
                                 ctypes.cast(shape, ctypes.c_void_p), ctypes.cast(ctypes.pointer(rank), ctypes.c_void_p)) == 0
    return name.value.decode(), dtype.value.decode(), list(shape[:rank.value])


def test_w4a16_text_is_recognised_and_described():
    rc, key, err = _inject(_src("input0:float16[4096], qweight:int32[512, 4096], scales:float16[32, 4096] -> my_result:float16[4096]", W4A16))
    assert rc == 0, err
    L = _lib.load()
    n_in, n_out, name = ctypes.c_int(0), ctypes.c_int(0), ctypes.create_string_buffer(64)
    assert L.ab200_module_info(key, ctypes.cast(ctypes.pointer(n_in), ctypes.c_void_p), ctypes.cast(ctypes.pointer(n_out), ctypes.c_void_p),
                               ctypes.cast(name, ctypes.c_void_p), 64) == 0
    assert (n_in.value, n_out.value, name.value.decode()) == (3, 1, "my_result")
    assert _tensor(key, 1) == ("qweight", "int32", [512, 4096])
    assert _tensor(key, 3) == ("my_result", "float16", [4096])
    # a second text gets its own key; the positional einstein_v2("...") form of older scripts is read too
    rc2, key2, err2 = _inject(_src("data:float32[1000] -> sigmoid_f32:float32[1000]", "x").replace(
        'einstein_v2(input_dict={}, extra_outputs=[], exprss="x")', 'einstein_v2("sigmoid_f32[N] = 1 - 1 / (1 + data[N].call(strs.exp))", input_dict={})'))
    assert rc2 == 0 and key2 != key, err2
    # forward() checks the argument count before anything touches the device
    args = (ctypes.c_void_p * 2)(0, 0)
    assert L.ab200_forward(key, ctypes.cast(args, ctypes.c_void_p), 2, None) == _lib.EINVAL
    assert L.ab200_forward(10 ** 6, ctypes.cast(args, ctypes.c_void_p), 2, None) == _lib.EINVAL


def test_softmax_and_canonical_sigmoid_forms():
    sm = ("temp0[N] >=! input0[N, C]; temp1[N] +=! (input0[N, C] - temp0[N]).call(`exp`); "
          "output0[N, C] = (input0[N, C] - temp0[N]).call(`exp`) / temp1[N]")
    rc, key, err = _inject(_src("input0:float16[32, 4096] -> output0:float16[32, 4096]", sm))
    assert rc == 0, err
    rc, key, err = _inject(_src("input0:float32[8, 16] -> output0:float32[8, 16]", "output0[N, M] = 1.0 / (1.0 + (-input0[N, M]).call(`exp`))"))
    assert rc == 0, err


@pytest.mark.parametrize("text,code", [
    (_src("a:float32[8] -> b:float32[8]", "b[N] = a[N] + 1", backend="c-cuda"), _lib.EUNSUPPORTED),        # another backend's text
    (_src("a:float32[8, 8], c:float32[8, 8] -> b:float32[8, 8]", "b[N, M] +=! a[N, K] * c[K, M]"), _lib.EUNSUPPORTED),  # no kernel for it
    (_src("input0:float16[4096], qweight:int32[512, 4096], scales:float16[16, 4096] -> my_result:float16[4096]", W4A16), _lib.EINVAL),  # scales rows
    (_src("input0:float16[4096], qweight:int32[512, 4096], scales:float32[32, 4096] -> my_result:float16[4096]", W4A16), _lib.EUNSUPPORTED),  # mixed dtypes
    ("// BACKEND: c-b200 (default)\n// COMPUTE_V1: - einstein_v2(exprss=\"b[N] = a[N]\")\n", _lib.EINVAL),  # no GLOBALS line
    (_src("a:float32[8] b:float32[8]", "b[N] = a[N]"), _lib.EINVAL),                                        # no ` -> `
])
def test_rejections_are_errors_not_fallbacks(text, code):
    rc, key, err = _inject(text)
    assert rc == code and err, (rc, err)

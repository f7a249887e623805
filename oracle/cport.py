"""numpy-facing wrappers of the plain-C oracle (oracle/antares_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU-baseline leg of the
benchmark; never by the product package.  fp16 arrays are numpy float16; the C side sees their
bit patterns.
"""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = ctypes.CDLL(path)
        L.orc_digest_f16.restype = ctypes.c_double
        L.orc_digest_f32.restype = ctypes.c_double
        L.orc_argmax_f32.restype = ctypes.c_long
        _lib = L
    return _lib


def _p(a):
    assert a.flags["C_CONTIGUOUS"], "oracle wants contiguous arrays"
    return ctypes.c_void_p(a.ctypes.data)


def _l(v):
    return ctypes.c_long(int(v))


def _f(v):
    return ctypes.c_float(float(v))


def w4_unpack(qweight):
    Kp, N = qweight.shape
    out = np.empty((Kp * 8, N), np.uint8)
    lib().orc_w4_unpack(_p(qweight), _l(Kp * 8), _l(N), _p(out))
    return out


def w4_pack(q):
    K, N = q.shape
    assert K % 8 == 0
    q = np.ascontiguousarray(q, np.uint8)
    out = np.empty((K // 8, N), np.int32)
    lib().orc_w4_pack(_p(q), _l(K), _l(N), _p(out))
    return out


def w4_dequant(qweight, scales, group=128):
    Kp, N = qweight.shape
    K = Kp * 8
    if scales.dtype == np.float16:
        out = np.empty((K, N), np.float16)
        lib().orc_w4_dequant_f16(_p(qweight), _p(scales), _l(K), _l(N), _l(group), _p(out))
    else:
        out = np.empty((K, N), np.float32)
        lib().orc_w4_dequant_f32(_p(qweight), _p(scales), _l(K), _l(N), _l(group), _p(out))
    return out


def w4a16_gemm(x, qweight, scales, group=128):
    """x [M, K] (or [K]) fp16/fp32 -> [M, N] (or [N]) in x's dtype, fp32 accumulation."""
    squeeze = x.ndim == 1
    x2 = np.ascontiguousarray(x.reshape(1, -1) if squeeze else x)
    M, K = x2.shape
    Kp, N = qweight.shape
    assert Kp * 8 == K and scales.shape == (K // group, N)
    out = np.empty((M, N), x2.dtype)
    if x2.dtype == np.float16:
        assert scales.dtype == np.float16
        lib().orc_w4a16_gemm_f16(_p(x2), _p(qweight), _p(scales), _l(M), _l(K), _l(N), _l(group), _p(out))
    else:
        assert x2.dtype == np.float32 and scales.dtype == np.float32
        lib().orc_w4a16_gemm_f32(_p(x2), _p(qweight), _p(scales), _l(M), _l(K), _l(N), _l(group), _p(out))
    return out[0] if squeeze else out


def dense_gemv_f16(x, w):
    N, K = w.shape
    out = np.empty((N,), np.float32)
    lib().orc_dense_gemv_f16(_p(np.ascontiguousarray(x)), _p(w), _l(K), _l(N), _p(out))
    return out


def sigmoid(x):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    fn = lib().orc_sigmoid_f32 if x.dtype == np.float32 else lib().orc_sigmoid_f16
    fn(_p(x), _l(x.size), _p(out))
    return out


def rmsnorm(x, weight, eps=1e-6):
    """x [rows, cols] fp16 or fp32; weight fp16 [cols]; fp16 result."""
    x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
    rows, cols = x2.shape
    out = np.empty((rows, cols), np.float16)
    if x2.dtype == np.float32:
        lib().orc_rmsnorm_f32in_f16out(_p(x2), _p(weight), _l(rows), _l(cols), _f(eps), _p(out))
    else:
        lib().orc_rmsnorm_f16(_p(x2), _p(weight), _l(rows), _l(cols), _f(eps), _p(out))
    return out.reshape(x.shape)


def rmsnorm_vsum_f32(x, vsum, weight, inv_n, eps=1e-6):
    out = np.empty_like(x)
    lib().orc_rmsnorm_vsum_f32(_p(x), _p(vsum), _p(weight), _l(x.size), _f(inv_n), _f(eps), _p(out))
    return out


def make_inv_freq(D, base=10000.0):
    """Length-D fp32 table, two equal halves (samples/05_llama2_7b_int4.py:125-126)."""
    j = np.arange(0, D, 2, dtype=np.float32)
    f = (1.0 / (np.float32(base) ** (j / np.float32(D)))).astype(np.float32)
    return np.concatenate([f, f]).astype(np.float32)


def rope(x, pos, inv_freq):
    """x [rows, H, D] fp16; pos int32 [rows]."""
    x = np.ascontiguousarray(x)
    rows, H, D = x.shape
    pos = np.ascontiguousarray(pos, np.int32)
    out = np.empty_like(x)
    lib().orc_rope_f16(_p(x), _p(np.ascontiguousarray(inv_freq, np.float32)), _p(pos), _l(rows), _l(H), _l(D), _p(out))
    return out


def softmax(x):
    x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
    out = np.empty_like(x2)
    fn = lib().orc_softmax_f16 if x2.dtype == np.float16 else lib().orc_softmax_f32
    fn(_p(x2), _l(x2.shape[0]), _l(x2.shape[1]), _p(out))
    return out.reshape(x.shape)


def attention_decode(q, kc, vc, S, scale):
    """q [H, D]; kc, vc [>=S, H*D] fp16 cache rows (row stride = kc.shape[1])."""
    H, D = q.shape
    out = np.empty((H, D), np.float16)
    lib().orc_attention_decode_f16(_p(np.ascontiguousarray(q)), _p(kc), _p(vc), _l(S), _l(H), _l(D),
                                   _l(kc.shape[-1] if kc.ndim == 2 else H * D), _f(scale), _p(out))
    return out


def silu_mul(gate, up):
    out = np.empty_like(gate)
    lib().orc_silu_mul_f16(_p(np.ascontiguousarray(gate)), _p(np.ascontiguousarray(up)), _l(gate.size), _p(out))
    return out


def residual_add(x_f32, xb_f16):
    lib().orc_residual_add_f32(_p(x_f32), _p(np.ascontiguousarray(xb_f16)), _l(x_f32.size))
    return x_f32


def argmax(x):
    return int(lib().orc_argmax_f32(_p(np.ascontiguousarray(x, np.float32)), _l(x.size)))


def digest(x):
    x = np.ascontiguousarray(x)
    if x.dtype == np.float16:
        return float(lib().orc_digest_f16(_p(x), _l(x.size)))
    return float(lib().orc_digest_f32(_p(x.astype(np.float32)), _l(x.size)))


# ---- independent numpy restatement (guards the C text; small sizes only) -----------------------

def np_w4_unpack(qweight):
    Kp, N = qweight.shape
    sh = (np.arange(8, dtype=np.int32) * 4).reshape(1, 8, 1)
    return ((qweight.reshape(Kp, 1, N) >> sh) & 15).astype(np.uint8).reshape(Kp * 8, N)


def np_w4_dequant(qweight, scales, group=128):
    q = np_w4_unpack(qweight).astype(np.int32) - 8
    s = np.repeat(scales, group, axis=0)
    return (s * q.astype(scales.dtype)).astype(scales.dtype)


def np_w4a16_gemm(x, qweight, scales, group=128):
    w = np_w4_dequant(qweight, scales, group).astype(np.float32)
    y = x.astype(np.float32).reshape(-1, w.shape[0]) @ w
    return y.astype(x.dtype).reshape(x.shape[:-1] + (w.shape[1],))

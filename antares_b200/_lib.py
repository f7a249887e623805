"""ctypes binding of libantares_b200.so (the C ABI declared in include/antares_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libantares_b200.so")

OK, EINVAL, ECUDA, EUNSUPPORTED, ETIMEOUT = 0, 1, 2, 3, 4
F16, F32 = 0, 1


class Ab200Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__("antares_b200 error %d: %s" % (code, text))
        self.code = code


_vp, _i, _l, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_size_t

# name -> argument types; every function returns int except the two noted below.
SIGNATURES = {
    "ab200_device_info": [_i, _vp],
    "ab200_w4_unpack": [_vp, _i, _i, _vp, _vp],
    "ab200_w4_pack": [_vp, _i, _i, _vp, _vp],
    "ab200_w4_dequant": [_vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ab200_w4a16_gemv": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ab200_w4a16_gemv_residual": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ab200_w4a16_gemv_f32out": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ab200_w4a16_gemv_fused": [_vp, _i, _vp, _f, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "ab200_w4a16_gemv_static": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ab200_residual_add": [_vp, _vp, _i, _vp],
    "ab200_kernel_status": [_vp],
    "ab200_set_option": [ctypes.c_char_p, _i],
    "ab200_comm_alloc": [_i, _i, _vp, _vp],
    "ab200_comm_open": [_vp, _vp],
    "ab200_comm_close": [_vp],
    "ab200_comm_free": [_vp],
    "ab200_allreduce_residual": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "ab200_allreduce_residual_emulated": [_vp, _vp, _i, _vp, _i, _i, _vp, _vp],
    "ab200_w4a16_gemv_prefetch_hint": [_vp, _sz, _vp, _sz],
    "ab200_w4a16_gemv_tiled": [_vp, _i, _vp, _f, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ab200_eltwise_vm": [_vp, _vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _sz, _vp],
    "ab200_rowreduce_vm": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "ab200_embed_rows": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ab200_rope_kv_store_rows": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _l, _i, _vp],
    "ab200_attention_prefill": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _l, _f, _vp],
    "ab200_silu_mul_rows": [_vp, _vp, _i, _i, _vp],
    "ab200_residual_add_f16": [_vp, _vp, _sz, _vp],
    "ab200_greedy_next_tp_emulated": [_vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp],
    "ab200_greedy_next_tp": [_vp, _i, _i, _vp, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _i, _vp],
    "ab200_w4a16_gemv_tiled_allreduce": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _i, _vp],
    "ab200_w4a16_gemv_tiled_allreduce_emulated": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp, _vp],
    "ab200_w4a16_gemm": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ab200_sigmoid": [_vp, _vp, _sz, _i, _vp],
    "ab200_rmsnorm_vsum": [_vp, _vp, _vp, _vp, _sz, _f, _f, _i, _vp],
    "ab200_rmsnorm": [_vp, _i, _vp, _vp, _i, _i, _f, _vp],
    "ab200_rope": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ab200_softmax": [_vp, _vp, _i, _i, _i, _vp],
    "ab200_attention_decode": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _l, _f, _i, _vp],
    "ab200_embed_lookup": [_vp, _vp, _vp, _i, _i, _vp],
    "ab200_rope_kv_store": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _l, _i, _vp],
    "ab200_attention_fused": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _l, _i, _f, _vp],
    "ab200_attention_fused_paged": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _l, _i, _f, _vp, _i, _vp],
    "ab200_rope_kv_store_rows_paged": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _l, _i, _vp, _i, _vp],
    "ab200_attention_prefill_paged": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _l, _f, _vp, _i, _vp],
    "ab200_silu_mul": [_vp, _vp, _i, _vp],
    "ab200_dense_gemv": [_vp, _vp, _vp, _i, _i, _vp],
    "ab200_hal_set_device": [_i],
    "ab200_hal_malloc": [_vp, _sz],
    "ab200_hal_free": [_vp],
    "ab200_hal_memcpy": [_vp, _vp, _sz, _i, _vp],
    "ab200_hal_synchronize": [_vp],
    "ab200_hal_event_record": [_vp, _vp],
    "ab200_hal_event_elapsed": [_vp, _vp, _vp],
    "ab200_inject": [ctypes.c_char_p, _vp],
    "ab200_forward": [_i, _vp, _i, _vp],
    "ab200_module_info": [_i, _vp, _vp, _vp, _i],
    "ab200_module_tensor": [_i, _i, _vp, _i, _vp, _i, _vp, _vp],
    "ab200_forward_host_ns": [_i, _vp, _i, _vp, _i, _vp],
    "ab200_greedy_next": [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp],
}
OTHER_SYMBOLS = ["ab200_last_error", "ab200_abi_version", "ab200_w4a16_gemv_workspace_bytes", "ab200_comm_buffer_bytes",
                 "ab200_comm_emulation_scratch_bytes", "ab200_w4a16_gemv_emulation_scratch_bytes"]

_lib = None


def load():
    """Loads the library (once).  Raises ImportError if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not found: run `python -m antares_b200.build` (needs nvcc); "
                              "antares_b200 has no CPU or eager fallback" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        L.ab200_last_error.restype = ctypes.c_char_p
        L.ab200_last_error.argtypes = []
        L.ab200_abi_version.restype = ctypes.c_int
        L.ab200_w4a16_gemv_workspace_bytes.restype = ctypes.c_size_t
        L.ab200_w4a16_gemv_workspace_bytes.argtypes = [_i, _i, _i]
        L.ab200_comm_buffer_bytes.restype = ctypes.c_size_t
        L.ab200_comm_buffer_bytes.argtypes = [_i, _i]
        L.ab200_comm_emulation_scratch_bytes.restype = ctypes.c_size_t
        L.ab200_comm_emulation_scratch_bytes.argtypes = []
        L.ab200_w4a16_gemv_emulation_scratch_bytes.restype = ctypes.c_size_t
        L.ab200_w4a16_gemv_emulation_scratch_bytes.argtypes = []
        _lib = L
    return _lib


def call(name, *args):
    L = load()
    rc = getattr(L, name)(*args)
    if rc != OK:
        raise Ab200Error(rc, L.ab200_last_error().decode())

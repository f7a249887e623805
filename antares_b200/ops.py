"""torch-tensor front ends of the C ABI.  Tensors must live on a CUDA device; launches go to
torch's current stream (the reference launches on the NULL stream, frameworks/pytorch/main_ops.cc:44).
Nothing here computes on the CPU: a CPU tensor is an error, not a fallback.
"""
import torch

from . import _lib
from ._lib import F16, F32, call

_DT = {torch.float16: F16, torch.float32: F32}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor (antares_b200 has no CPU path)" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise ValueError("%s must be %s, got %s" % (name, dtype, t.dtype))
    return t.data_ptr()


def _code(dtype):
    try:
        return _DT[dtype]
    except KeyError:
        raise ValueError("dtype %s is outside the built kernel family (float16, float32)" % dtype)


def device_info(device=0):
    import ctypes
    buf = (ctypes.c_int * 8)()
    call("ab200_device_info", int(device), ctypes.cast(buf, ctypes.c_void_p))
    keys = ["sm_count", "smem_optin_bytes", "l2_bytes", "sm_clock_khz", "mem_clock_khz", "bus_width_bits", "cc", "max_threads"]
    return dict(zip(keys, list(buf)))


def w4_unpack(qweight):
    Kp, N = qweight.shape
    out = torch.empty((Kp * 8, N), dtype=torch.uint8, device=qweight.device)
    call("ab200_w4_unpack", _chk(qweight, "qweight", torch.int32), Kp * 8, N, out.data_ptr(), _stream())
    return out


def w4_pack(q):
    K, N = q.shape
    out = torch.empty((K // 8, N), dtype=torch.int32, device=q.device)
    call("ab200_w4_pack", _chk(q, "q", torch.uint8), K, N, out.data_ptr(), _stream())
    return out


def w4_dequant(qweight, scales, group=128):
    Kp, N = qweight.shape
    out = torch.empty((Kp * 8, N), dtype=scales.dtype, device=qweight.device)
    call("ab200_w4_dequant", _chk(qweight, "qweight", torch.int32), _chk(scales, "scales"), Kp * 8, N, group,
         _code(scales.dtype), out.data_ptr(), _stream())
    return out


def _gemm_shapes(x, qweight, scales, group):
    Kp, N = qweight.shape
    K = Kp * 8
    if x.shape[-1] != K:
        raise ValueError("x has %d features but qweight packs %d" % (x.shape[-1], K))
    M = x.numel() // K
    if group is None:
        group = K // scales.shape[0]
    if scales.shape != (K // group, N):
        raise ValueError("scales shape %s does not match [K/group=%d, N=%d]" % (tuple(scales.shape), K // group, N))
    if scales.dtype != x.dtype:
        raise ValueError("x (%s) and scales (%s) must share a dtype" % (x.dtype, scales.dtype))
    return M, K, N, group


def w4a16_gemv(x, qweight, scales, out=None, group=None):
    """out[..., N] = x[..., K] . dequant(qweight, scales); M = x.numel()/K <= 16."""
    M, K, N, group = _gemm_shapes(x, qweight, scales, group)
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=x.dtype, device=x.device)
    elif out.numel() != M * N or out.dtype != x.dtype:
        raise ValueError("out must hold %d elements of %s" % (M * N, x.dtype))
    call("ab200_w4a16_gemv", _chk(x, "x"), _chk(qweight, "qweight", torch.int32), _chk(scales, "scales"),
         _chk(out, "out"), M, K, N, group, _code(x.dtype), _stream())
    return out


def w4a16_gemv_residual(x, qweight, scales, resid, group=None):
    """resid_f32[..., N] += fp16_round(x . W)."""
    M, K, N, group = _gemm_shapes(x, qweight, scales, group)
    if resid.numel() != M * N:
        raise ValueError("resid must hold %d elements" % (M * N))
    call("ab200_w4a16_gemv_residual", _chk(x, "x", torch.float16), _chk(qweight, "qweight", torch.int32),
         _chk(scales, "scales", torch.float16), _chk(resid, "resid", torch.float32), M, K, N, group, _stream())
    return resid


def w4a16_gemm(x, qweight, scales, out=None, group=None):
    """Prefill contraction on tensor cores; x [M, K] with M a multiple of 128."""
    Kp, N = qweight.shape
    K = Kp * 8
    M = x.numel() // K
    if group is None:
        group = K // scales.shape[0]
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=x.dtype, device=x.device)
    call("ab200_w4a16_gemm", _chk(x, "x"), _chk(qweight, "qweight", torch.int32), _chk(scales, "scales"),
         _chk(out, "out"), M, K, N, group, _code(x.dtype), _stream())
    return out


def w4a16_matmul(x, qweight, scales, out=None, group=None):
    """The exported op of samples/05_llama2_7b_int4.py:135-144 for any batch: decode kernel up to
    16 rows, tensor-core kernel above."""
    M = x.numel() // (qweight.shape[0] * 8)
    if M <= 16:
        return w4a16_gemv(x, qweight, scales, out, group)
    return w4a16_gemm(x, qweight, scales, out, group)


def sigmoid(x, out=None):
    if out is None:
        out = torch.empty_like(x)
    call("ab200_sigmoid", _chk(x, "x"), _chk(out, "out", x.dtype), x.numel(), _code(x.dtype), _stream())
    return out


def rmsnorm_vsum(x, vsum, weight, inv_n, eps=1e-6, out=None):
    if out is None:
        out = torch.empty_like(x)
    call("ab200_rmsnorm_vsum", _chk(x, "x"), _chk(vsum, "vsum", torch.float32), _chk(weight, "weight", x.dtype),
         _chk(out, "out", x.dtype), x.numel(), float(inv_n), float(eps), _code(x.dtype), _stream())
    return out


def rmsnorm(x, weight, eps=1e-6, out=None):
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    call("ab200_rmsnorm", _chk(x, "x"), _code(x.dtype), _chk(weight, "weight", torch.float16),
         _chk(out, "out", torch.float16), rows, cols, float(eps), _stream())
    return out


def rope(x, pos, inv_freq, out=None):
    rows, H, D = x.shape
    if out is None:
        out = torch.empty_like(x)
    call("ab200_rope", _chk(x, "x"), _chk(inv_freq, "inv_freq", torch.float32),
         _chk(pos, "pos", torch.int32), _chk(out, "out", x.dtype), rows, H, D, _code(x.dtype), _stream())
    return out


def softmax(x, out=None):
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    call("ab200_softmax", _chk(x, "x"), _chk(out, "out", x.dtype), rows, cols, _code(x.dtype), _stream())
    return out


def attention_decode(q, k_cache, v_cache, seq_len_dev, scale, out=None, kv_stride=None, max_seq=None, seq_len_add=0):
    H, D = q.shape
    if kv_stride is None:
        kv_stride = k_cache.stride(0)
    if max_seq is None:
        max_seq = k_cache.shape[0]
    if out is None:
        out = torch.empty_like(q)
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("q, k_cache and v_cache must share a dtype")
    call("ab200_attention_decode", _chk(q, "q"), k_cache.data_ptr(), v_cache.data_ptr(),
         _chk(out, "out", q.dtype), _chk(seq_len_dev, "seq_len_dev", torch.int32), int(seq_len_add), int(max_seq), H, D,
         int(kv_stride), float(scale), _code(q.dtype), _stream())
    return out


def set_option(name, value):
    """Process-wide tuning knob (gemv_cluster, gemv_impl)."""
    call("ab200_set_option", name.encode(), int(value))


def kernel_status():
    """Reads and clears the device status word; raises Ab200Error(ETIMEOUT) if a bounded wait ran out."""
    import ctypes
    v = ctypes.c_int(0)
    call("ab200_kernel_status", ctypes.cast(ctypes.pointer(v), ctypes.c_void_p))
    return v.value


PRO_PLAIN, PRO_RMSNORM, PRO_SILU_MUL = 0, 1, 2
EPI_F16, EPI_RESIDUAL, EPI_F32 = 0, 1, 2


def gemv_workspace_bytes(M, K, N):
    return int(_lib.load().ab200_w4a16_gemv_workspace_bytes(int(M), int(K), int(N)))


def w4a16_gemv_fused(x, qweight, scales, out, prologue=PRO_PLAIN, epilogue=EPI_F16, norm_weight=None, eps=1e-6,
                     group=None, workspace=None):
    """One-launch decode projection: optional RMSNorm / SiLU*up on the way in, optional residual
    add on the way out.  x: fp16 [M,K] (plain), fp32 [M,K] (RMSNorm) or fp16 [M,2K] (SiLU*up)."""
    Kp, N = qweight.shape
    K = Kp * 8
    xk = 2 * K if prologue == PRO_SILU_MUL else K
    M = x.numel() // xk
    if group is None:
        group = K // scales.shape[0]
    want_x = torch.float32 if prologue == PRO_RMSNORM else torch.float16
    want_o = torch.float16 if epilogue == EPI_F16 else torch.float32
    if out.numel() != M * N:
        raise ValueError("out must hold %d elements" % (M * N))
    ws_ptr, ws_bytes = (0, 0) if workspace is None else (_chk(workspace, "workspace"), workspace.numel() * workspace.element_size())
    call("ab200_w4a16_gemv_fused", _chk(x, "x", want_x), int(prologue),
         0 if norm_weight is None else _chk(norm_weight, "norm_weight", torch.float16), float(eps),
         _chk(qweight, "qweight", torch.int32), _chk(scales, "scales", torch.float16), _chk(out, "out", want_o), int(epilogue),
         M, K, N, group, ws_ptr, ws_bytes, _stream())
    return out


def w4a16_gemv_tiled(x, qweight_tiled, scales_tiled, out, prologue=PRO_PLAIN, epilogue=EPI_F16, norm_weight=None, eps=1e-6, group=128):
    """w4a16_gemv_fused on tile-major weights (packing.tile_weights): qweight_tiled [N/128, K/8, 128]."""
    K, N = qweight_tiled.shape[1] * 8, qweight_tiled.shape[0] * qweight_tiled.shape[2]
    xk = x.shape[-1] // 2 if prologue == PRO_SILU_MUL else x.shape[-1]
    if xk != K:
        raise ValueError("x has %d values per row, the weights %d rows" % (xk, K))
    M = x.numel() // x.shape[-1]
    call("ab200_w4a16_gemv_tiled", _chk(x, "x"), prologue, 0 if norm_weight is None else _chk(norm_weight, "norm_weight", torch.float16), float(eps),
         _chk(qweight_tiled, "qweight_tiled", torch.int32), _chk(scales_tiled, "scales_tiled", torch.float16), _chk(out, "out"),
         epilogue, M, K, N, group, _stream())
    return out


def eltwise_program(prog, consts, inputs, out=None, out_dtype=None):
    """Runs a stack program (ir.compile_elementwise) over same-sized fp16/fp32 tensors."""
    import ctypes
    n = inputs[0].numel()
    for t in inputs:
        if t.numel() != n:
            raise ValueError("element-wise inputs must all hold %d elements" % n)
    if out is None:
        out = torch.empty_like(inputs[0], dtype=out_dtype or inputs[0].dtype)
    elif out.numel() != n:
        raise ValueError("out must hold %d elements" % n)
    ops_b = (ctypes.c_ubyte * len(prog))(*[int(o) for o, _ in prog])
    args_b = (ctypes.c_ubyte * len(prog))(*[int(a) for _, a in prog])
    cst = (ctypes.c_float * max(1, len(consts)))(*[float(c) for c in consts])
    ptrs = (ctypes.c_void_p * len(inputs))(*[_chk(t, "input") for t in inputs])
    dts = (ctypes.c_int * len(inputs))(*[_code(t.dtype) for t in inputs])
    call("ab200_eltwise_vm", ctypes.cast(ops_b, ctypes.c_void_p), ctypes.cast(args_b, ctypes.c_void_p), len(prog), ctypes.cast(cst, ctypes.c_void_p),
         len(consts), ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(dts, ctypes.c_void_p), len(inputs), _chk(out, "out"), _code(out.dtype), n, _stream())
    return out


def row_program(rp, mats, cols, out=None, out_dtype=None):
    """Runs a compiled reduce + map chain (ir.compile_row_program) over [..., cols] tensors: `mats` the
    full-shape inputs, `cols` the [cols] vectors, in the program's operand order."""
    import ctypes
    shape = mats[0].shape
    ncols = shape[-1]
    rows = mats[0].numel() // ncols
    for t in mats:
        if t.shape != shape:
            raise ValueError("row program: full-shape inputs must share one shape (%s vs %s)" % (tuple(t.shape), tuple(shape)))
    for t in cols:
        if t.numel() != ncols:
            raise ValueError("row program: a column vector must hold %d elements" % ncols)
    if out is None:
        dt = out_dtype or (torch.float32 if any(a.dtype == torch.float32 for a in list(mats) + list(cols)) else torch.float16)
        out = torch.empty(shape, dtype=dt, device=mats[0].device)
    elif out.numel() != mats[0].numel():
        raise ValueError("out must hold %d elements" % mats[0].numel())
    flat = [oa for _, prog in rp["stages"] for oa in prog]
    ops_b = (ctypes.c_ubyte * len(flat))(*[int(o) for o, _ in flat])
    args_b = (ctypes.c_ubyte * len(flat))(*[int(a) for _, a in flat])
    lens = (ctypes.c_int * len(rp["stages"]))(*[len(prog) for _, prog in rp["stages"]])
    kinds = (ctypes.c_int * len(rp["stages"]))(*[int(k) for k, _ in rp["stages"]])
    consts = rp["consts"]
    cst = (ctypes.c_float * max(1, len(consts)))(*[float(c) for c in consts])
    mp = (ctypes.c_void_p * len(mats))(*[_chk(t, "input") for t in mats])
    md = (ctypes.c_int * len(mats))(*[_code(t.dtype) for t in mats])
    cp = (ctypes.c_void_p * max(1, len(cols)))(*[_chk(t, "column vector") for t in cols])
    cd = (ctypes.c_int * max(1, len(cols)))(*[_code(t.dtype) for t in cols])
    P = ctypes.c_void_p
    call("ab200_rowreduce_vm", ctypes.cast(ops_b, P), ctypes.cast(args_b, P), ctypes.cast(lens, P), ctypes.cast(kinds, P), len(rp["stages"]),
         ctypes.cast(cst, P), len(consts), ctypes.cast(mp, P), ctypes.cast(md, P), len(mats), ctypes.cast(cp, P), ctypes.cast(cd, P), len(cols),
         _chk(out, "out"), _code(out.dtype), rows, ncols, _stream())
    return out

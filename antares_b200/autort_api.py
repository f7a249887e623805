"""The AutoRT calling surface, kept so that scripts written for the reference run on the B200
kernel library unchanged.

Reference usage (the AutoRT package itself ships only as a wheel; call sites are in-tree):
  f = autort.export(ir=..., inputs=["name=dtype[Dim:val, ...]"], config=..., name=...)   README.md:63-69
  f(x, qweight, scales, out=buf)            samples/05_llama2_7b_int4.py:135-144
  autort.ops.rmsnorm_f32(x, vsum, w, extra=[1/N])                  samples/05_llama2_7b_int4.py:128-131
  autort.ops.rotary_f32(x.view(H,2,-1), inv_freq, out, extra=[pos])  samples/05_llama2_7b_int4.py:157-158
  autort.ops.attention_f32(q, k, v, att_f)                           samples/05_llama2_7b_int4.py:161-165
  autort.device()                                                    samples/05_llama2_7b_int4.py:78

Calling convention kept: tensors positionally in declared order; the result is returned, or
written into a trailing positional tensor / `out=`; scalars come through `extra=[...]`; dimensions
declared `Name:val` are upper bounds, the call may pass fewer elements (README.md:64-67).
`config=` carries tuner hints in the reference ("tune:5", "~N~:[256,8,32],..."): the kernels here
are hand-scheduled, so it is accepted and ignored.  Outside the named family, single element-wise
statements run on a generic interpreter kernel (ir.compile_elementwise) and chains of row reductions
closed by one map statement (layernorm and the like) on the row-reduction template
(ir.compile_row_program); other IR raises NotImplementedError; nothing runs on the CPU.
"""
import torch

from . import ir as _ir
from . import ops as _ops

RMS_EPS = 1e-6  # epsilon of the built-in rmsnorm ops (the reference's value is inside its closed wheel)

# The W4A16 program of the reference's int4 sample (samples/05_llama2_7b_int4.py:136-138), for callers that
# want the exported op without retyping the IR.
W4A16_IR_SAMPLE = """
  input1[S, N] = (qweight[S / 8, N] >> (S % 8 * 4)).call(strs.bitwise_and, 15) * input0[S].like(1)
  w[S, N] = scales[S / 128, N] * (input1[S, N] - 8)
  my_result[N] +=! input0[S] * w[S, N].to(input0.dtype())
"""

_TORCH_DT = {"float16": torch.float16, "float32": torch.float32, "int32": torch.int32}


def device():
    """The device custom ops run on (samples/05_llama2_7b_int4.py:78)."""
    if not torch.cuda.is_available():
        raise RuntimeError("antares_b200 needs a CUDA device: there is no CPU backend")
    return torch.device("cuda", torch.cuda.current_device())


class _OpNamespace:
    """autort.ops.<name>: ops registered by export() plus the built-in Llama ops."""

    def _register(self, name, fn):
        setattr(self, name, fn)


ops = _OpNamespace()


def _split_call(match, tensors, out):
    """Positional tensors = declared inputs [+ output].  Returns (inputs by name, out)."""
    n_in = len(match.inputs)
    if len(tensors) == n_in + 1 and out is None:
        tensors, out = tensors[:n_in], tensors[n_in]
    if len(tensors) != n_in:
        raise TypeError("%s expects %d tensors (%s)%s, got %d" % (match.name, n_in, ", ".join(s.name for s in match.inputs),
                                                                  " plus an optional output", len(tensors)))
    by_name = {}
    for spec, t in zip(match.inputs, tensors):
        want = _TORCH_DT.get(spec.dtype)
        if want is not None and t.dtype != want:
            raise TypeError("%s: tensor %s must be %s, got %s" % (match.name, spec.name, spec.dtype, t.dtype))
        if t.dim() != len(spec.dims):
            raise ValueError("%s: tensor %s must have %d dimensions" % (match.name, spec.name, len(spec.dims)))
        for size, bound, dyn in zip(t.shape, spec.dims, spec.dyn):
            if (dyn is None and size != bound) or size > bound:
                raise ValueError("%s: tensor %s has extent %d where %s%d is declared" % (match.name, spec.name, size, "at most " if dyn else "", bound))
        by_name[spec.name] = t.contiguous()
    return by_name, out


class NativeModules:
    """Keys of the library's native plugin boundary (ab200_inject / ab200_forward, the counterpart of
    frameworks/pytorch/main_ops.cc:17-54) for one exported op: the kernel-source text is written in the
    reference's wire format for the shapes of a call, injected once per distinct shape set, and every call
    goes through ab200_forward with raw pointers - the same entry a C++ binding would use, so there is one
    recogniser for both routes (the IR is matched natively; Python only formats the header)."""

    def __init__(self, ir_text, input_specs, out_name):
        self.ir = "; ".join(_ir.split_statements(ir_text))
        self.specs, self.out_name = input_specs, out_name
        self.order = sorted(range(len(input_specs)), key=lambda i: input_specs[i].name)  # inputs sorted by name (lang/generic.py:53-54)
        self.keys = {}

    def source(self, shapes, out_dtype, out_shape):
        ins = ", ".join("%s:%s[%s]" % (self.specs[i].name, self.specs[i].dtype, ", ".join(str(d) for d in shapes[i])) for i in self.order)
        outs = "%s:%s[%s]" % (self.out_name, out_dtype, ", ".join(str(d) for d in out_shape))
        return ("// GLOBALS: %s -> %s\n// BACKEND: c-b200 (default)\n// CONFIG: \n// COMPUTE_V1: - einstein_v2(input_dict={}, extra_outputs=[], exprss=\"%s\")\n"
                % (ins, outs, self.ir))

    def forward(self, tensors, out, out_dtype_name):
        import ctypes
        from ._lib import call
        shapes = tuple(tuple(t.shape) for t in tensors)
        sig = (shapes, tuple(out.shape))
        key = self.keys.get(sig)
        if key is None:
            k = ctypes.c_int(-1)
            call("ab200_inject", self.source(shapes, out_dtype_name, tuple(out.shape)).encode(), ctypes.cast(ctypes.pointer(k), ctypes.c_void_p))
            key = self.keys[sig] = k.value
        n = len(tensors) + 1
        args = (ctypes.c_void_p * n)(*([tensors[i].data_ptr() for i in self.order] + [out.data_ptr()]))
        call("ab200_forward", key, ctypes.cast(args, ctypes.c_void_p), n, torch.cuda.current_stream().cuda_stream)
        return out


_DT_NAME = {torch.float16: "float16", torch.float32: "float32"}


def export(ir, inputs, config=None, name=None):
    """Binds an Antares-IR program to its hand-written kernel and registers it as autort.ops.<name>."""
    match = _ir.recognise(ir, inputs, name)
    if match.kind in ("w4a16", "sigmoid", "softmax"):
        pr = match.params
        native = NativeModules(ir, match.inputs, match.output)

        def fn(*tensors, out=None, extra=None):
            t, out = _split_call(match, tensors, out)
            ordered = [t[s.name] for s in match.inputs]
            for a in ordered:
                if not a.is_cuda:
                    raise ValueError("%s: tensors must live on a CUDA device (there is no CPU path)" % match.name)
            x = t[pr["x"]]
            if match.kind == "w4a16":
                qw = t[pr["qweight"]]
                shape = tuple(x.shape[:-1]) + (qw.shape[1],)
            else:
                shape = tuple(x.shape)
            if out is None:
                out = torch.empty(shape, dtype=x.dtype, device=x.device)
            elif out.numel() != int(torch.Size(shape).numel()) or out.dtype != x.dtype or not out.is_contiguous():
                raise ValueError("%s: out must be a contiguous %s tensor of %d elements" % (match.name, x.dtype, torch.Size(shape).numel()))
            native.forward(ordered, out.view(shape) if out.shape != shape else out, _DT_NAME[x.dtype])
            return out
        fn.native = native
    elif match.kind == "eltwise":
        pr = match.params

        def fn(*tensors, out=None, extra=None):
            t, out = _split_call(match, tensors, out)
            ins = [t[n] for n in pr["inputs"]]
            shape = ins[0].shape
            for n, a in zip(pr["inputs"], ins):
                if a.shape != shape:
                    raise ValueError("%s: element-wise inputs must have one shape (%s has %s, expected %s)" % (match.name, n, tuple(a.shape), tuple(shape)))
            if out is None:
                # result dtype: the widest input dtype, as the reference's promotion rule gives (lang/einstein_v2.py:26-32)
                dt = torch.float32 if any(a.dtype == torch.float32 for a in ins) else torch.float16
                out = torch.empty(shape, dtype=dt, device=ins[0].device)
            return _ops.eltwise_program(pr["program"], pr["consts"], ins, out=out)
    elif match.kind == "rowprog":
        rp = match.params

        def fn(*tensors, out=None, extra=None):
            t, out = _split_call(match, tensors, out)
            return _ops.row_program(rp, [t[n] for n in rp["mats"]], [t[n] for n in rp["cols"]], out=out)
    else:  # pragma: no cover - recognise() raises first
        raise NotImplementedError(match.kind)
    fn.__name__ = match.name
    fn.match = match
    ops._register(match.name, fn)
    return fn


# ---- built-in ops of the Llama samples (closed in the reference; definitions in the oracle) ----------

def _rmsnorm(dtype):
    def fn(x, vsum, weight, out=None, extra=None):
        if not extra:
            raise TypeError("rmsnorm needs extra=[1/N]")
        if x.dtype != dtype or weight.dtype != dtype:
            raise TypeError("rmsnorm_%s: x and weight must be %s" % ("f32" if dtype == torch.float32 else "f16", dtype))
        return _ops.rmsnorm_vsum(x.contiguous(), vsum.reshape(1).float(), weight.contiguous(), float(extra[0]), RMS_EPS, out=out)
    return fn


def _rotary(dtype):
    def fn(x, inv_freq, out=None, extra=None):
        if not extra:
            raise TypeError("rotary needs extra=[pos]")
        if x.dtype != dtype:
            raise TypeError("rotary: x must be %s" % dtype)
        H = x.shape[0]
        D = x.numel() // H                      # x arrives as [H, 2, D/2]: the same memory as [H, D]
        pos = torch.tensor([int(extra[0])], dtype=torch.int32, device=x.device)
        res = _ops.rope(x.contiguous().view(1, H, D), pos, inv_freq.float().contiguous(),
                        out=None if out is None else out.view(1, H, D))
        return res.view(H, D) if out is None else out
    return fn


def _attention(dtype):
    def fn(q, k, v, att_f, out=None, extra=None):
        if q.dtype != dtype:
            raise TypeError("attention: q must be %s" % dtype)
        H, D = q.shape
        S = k.shape[0]                           # caches arrive narrowed to the rows to attend (line 162)
        seq = torch.tensor([S], dtype=torch.int32, device=q.device)
        return _ops.attention_decode(q.contiguous(), k, v, seq, float(att_f.reshape(-1)[0]), out=out,
                                     kv_stride=k.stride(0), max_seq=S)
    return fn


for _suffix, _dt in (("f32", torch.float32), ("f16", torch.float16)):
    ops._register("rmsnorm_" + _suffix, _rmsnorm(_dt))
    ops._register("rotary_" + _suffix, _rotary(_dt))
    ops._register("attention_" + _suffix, _attention(_dt))

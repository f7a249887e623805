"""`CustomOp`, the reference's legacy PyTorch binding (frameworks/pytorch/custom_op.py:39-148), on
the B200 kernel library.

Same constructor and call protocol: CustomOp(ir, input_orders={name: tensor | (_, dtype, shape)},
extra_outputs=[], device=...).tune().emit(); op(*inputs) -> tensor.  Where the reference shells
out to its compiler for kernel text and JIT-compiles it, emit() here binds the IR to a
precompiled kernel (antares_b200.ir.recognise); tune() has nothing to search and returns self.
Inputs are taken in the order of `input_orders`, as the reference's forward() does
(custom_op.py:136-140); outputs are allocated with torch.empty.
"""
import torch

from . import ir as _ir
from . import ops as _ops

_DT_NAME = {torch.float16: "float16", torch.float32: "float32", torch.int32: "int32", torch.float64: "float64",
            torch.int64: "int64", torch.int16: "int16", torch.int8: "int8"}


class CustomOp(torch.nn.Module):
    def __init__(self, ir, input_orders, extra_outputs=[], device=None):
        super().__init__()
        # the reference joins lines with spaces (custom_op.py:43) and so needs ';' between statements;
        # here newlines separate statements as well
        self.ir = ir.replace('"', "`").strip()
        self.input_names = list(input_orders)
        self.specs = []
        for k in self.input_names:
            v = input_orders[k]
            shape, dtype = (v[2], v[1]) if isinstance(v, tuple) else (v.shape, v.dtype)
            self.specs.append(_ir.TensorSpec(k, _DT_NAME[dtype], [int(d) for d in shape], [None] * len(shape)))
        if extra_outputs:
            raise NotImplementedError("extra_outputs are outside the hand-written operator family")
        self.custom_device = torch.device("cuda") if device is None else device
        if self.custom_device.type != "cuda":
            raise RuntimeError("antares_b200 has no CPU backend (the reference's c-mcpu path is only used as the test oracle)")
        self.match = None

    def tune(self, step=100, use_cache=False, timeout=-1):
        return self

    def emit(self):
        self.match = _ir.recognise(self.ir, self.specs)
        if self.match.kind in ("w4a16", "sigmoid", "softmax"):
            # the named family goes through the native plugin boundary (ab200_inject / ab200_forward), as the
            # reference's forward() goes through custom_lib.inject / custom_lib.forward (custom_op.py:117-148)
            from .autort_api import NativeModules
            self.native = NativeModules(self.ir, self.match.inputs, self.match.output)
        return self

    def forward(self, *inputs):
        if self.match is None:
            raise RuntimeError("call emit() before the first forward()")
        if len(inputs) != len(self.input_names):
            raise TypeError("expected %d inputs" % len(self.input_names))
        t = {k: v.contiguous().to(self.custom_device) for k, v in zip(self.input_names, inputs)}
        pr = self.match.params
        if self.match.kind in ("w4a16", "sigmoid", "softmax"):
            x = t[pr["x"]]
            shape = tuple(x.shape[:-1]) + (t[pr["qweight"]].shape[1],) if self.match.kind == "w4a16" else tuple(x.shape)
            out = torch.empty(shape, dtype=x.dtype, device=x.device)
            dt = {torch.float16: "float16", torch.float32: "float32"}[x.dtype]
            return self.native.forward([t[s.name] for s in self.match.inputs], out, dt)
        if self.match.kind == "eltwise":
            ins = [t[n] for n in pr["inputs"]]
            dt = torch.float32 if any(a.dtype == torch.float32 for a in ins) else torch.float16
            return _ops.eltwise_program(pr["program"], pr["consts"], ins, out=torch.empty(ins[0].shape, dtype=dt, device=ins[0].device))
        if self.match.kind == "rowprog":
            return _ops.row_program(pr, [t[n] for n in pr["mats"]], [t[n] for n in pr["cols"]])
        raise NotImplementedError(self.match.kind)

"""Recogniser for the Antares-IR programs on the Llama-2-7B int4 path.

The reference turns IR text into kernels with a general compiler (lang/einstein_v2.py:297-578 ->
antares/default_codegen.py).  This module does not compile: it parses the `inputs=` declarations
of `autort.export` (README.md:63-69, samples/05_llama2_7b_int4.py:135-139), normalises the IR text
with the reference's conventions, and matches it against the operator family that has a
hand-written sm_100a kernel.  Anything else raises NotImplementedError (there is no fallback).

Conventions kept from the reference:
  * statements are separated by newlines or ';' (frameworks/pytorch/custom_op.py:43 joins lines);
    `+=!` and `+=` are the same reduction (lang/einstein_v2.py:298);
  * upper-case identifiers are axes, lower-case ones tensors (lang/einstein_v2.py:9-10);
  * a shape entry `Name:val` declares a dynamic axis with upper bound val (lang/einstein_v2.py:524-535);
  * the op's name defaults to the l-value of the last statement (README.md:66-69).
"""
import re
from dataclasses import dataclass, field

DTYPES = ("float64", "float32", "float16", "int64", "int32", "int16", "int8")


@dataclass
class TensorSpec:
    name: str
    dtype: str
    dims: list          # upper bounds (ints)
    dyn: list           # axis name for dynamic dims, else None


@dataclass
class OpMatch:
    kind: str                       # "w4a16" | "sigmoid" | "softmax"
    name: str                       # exported op name
    inputs: list                    # TensorSpec in declared order
    output: str                     # l-value tensor of the last statement
    params: dict = field(default_factory=dict)


def parse_input_spec(text):
    """'input0=float32[S:4096]' -> TensorSpec(name, dtype, dims, dyn)."""
    m = re.fullmatch(r"\s*([A-Za-z_]\w*)\s*=\s*([a-z]+\d+)\s*\[(.*)\]\s*", text)
    if not m:
        raise ValueError("cannot parse input declaration %r (want name=dtype[dims])" % text)
    name, dtype, dims_text = m.groups()
    if dtype not in DTYPES:
        raise ValueError("unknown dtype %r in %r" % (dtype, text))
    dims, dyn = [], []
    for d in [t.strip() for t in dims_text.split(",") if t.strip()]:
        if ":" in d:
            axis, val = d.split(":")
            dims.append(int(val))
            dyn.append(axis.strip())
        else:
            dims.append(int(d))
            dyn.append(None)
    return TensorSpec(name, dtype, dims, dyn)


def split_statements(ir):
    ir = ir.replace('"', "`")
    parts = re.split(r"[;\n]", ir)
    return [re.sub(r"\s+", " ", p).strip() for p in parts if p.strip()]


def _squash(s):
    return re.sub(r"\s+", "", s).replace("+=!", "+=").replace(">=!", ">=")


def _lvalue(stmt):
    m = re.match(r"\s*([a-z_]\w*)\s*\[", stmt)
    if not m:
        raise ValueError("statement has no tensor l-value: %r" % stmt)
    return m.group(1)


# -- patterns (on whitespace-free text; tensor/axis names captured) ------------------------------------
_W4_S1 = re.compile(r"^(\w+)\[(\w+),(\w+)\]=\((\w+)\[\2/8,\3\]>>\(\2%8\*4\)\)\.call\(strs\.bitwise_and,15\)\*(\w+)\[\2\]\.like\(1\)$")
_W4_S2 = re.compile(r"^(\w+)\[(\w+),(\w+)\]=(\w+)\[\2/(\d+),\3\]\*\((\w+)\[\2,\3\]-8\)$")
_W4_S3 = re.compile(r"^(\w+)\[(\w+)\]\+=(\w+)\[(\w+)\]\*(\w+)\[\4,\2\]\.to\(\3\.dtype\(\)\)$")
_SIG_README = re.compile(r"^(\w+)\[(\w+)\]=1-1/\(1\+(\w+)\[\2\]\.call\(strs\.exp\)\)$")
_SIG_CANON = re.compile(r"^(\w+)\[([\w,]+)\]=1\.0/\(1\.0\+\(-(\w+)\[\2\]\)\.call\(`exp`\)\)$")
_SM_1 = re.compile(r"^(\w+)\[(\w+)\]>=(\w+)\[\2,(\w+)\]$")
_SM_2 = re.compile(r"^(\w+)\[(\w+)\]\+=\((\w+)\[\2,(\w+)\]-(\w+)\[\2\]\)\.call\(`exp`\)$")
_SM_3 = re.compile(r"^(\w+)\[(\w+),(\w+)\]=\((\w+)\[\2,\3\]-(\w+)\[\2\]\)\.call\(`exp`\)/(\w+)\[\2\]$")


def recognise(ir, inputs, name=None):
    """Returns an OpMatch or raises NotImplementedError."""
    specs = [parse_input_spec(t) if isinstance(t, str) else t for t in inputs]
    stmts = split_statements(ir)
    if not stmts:
        raise ValueError("empty IR")
    sq = [_squash(s) for s in stmts]
    out = _lvalue(stmts[-1])
    op_name = name or out
    by_name = {s.name: s for s in specs}

    if len(sq) == 3:
        m1, m2, m3 = _W4_S1.match(sq[0]), _W4_S2.match(sq[1]), _W4_S3.match(sq[2])
        if m1 and m2 and m3:
            nib, _, _, qweight, x1 = m1.groups()
            w, _, _, scales, group, nib2 = m2.groups()
            res, _, x3, _, w3 = m3.groups()
            if nib2 == nib and w3 == w and x1 == x3 and {qweight, scales, x1} <= set(by_name):
                if by_name[qweight].dtype != "int32":
                    raise NotImplementedError("W4A16: packed weights must be int32")
                if by_name[x1].dtype != by_name[scales].dtype or by_name[x1].dtype not in ("float16", "float32"):
                    raise NotImplementedError("W4A16: activations and scales must both be float16 or both float32")
                return OpMatch("w4a16", op_name, specs, res,
                               dict(x=x1, qweight=qweight, scales=scales, group=int(group), dtype=by_name[x1].dtype))
        m1, m2, m3 = _SM_1.match(sq[0]), _SM_2.match(sq[1]), _SM_3.match(sq[2])
        if m1 and m2 and m3 and m1.group(3) == m2.group(3) == m3.group(4) and m2.group(5) == m1.group(1) == m3.group(5) \
                and m3.group(6) == m2.group(1) and m1.group(3) in by_name:
            return OpMatch("softmax", op_name, specs, m3.group(1), dict(x=m1.group(3), dtype=by_name[m1.group(3)].dtype))
    if len(sq) == 1:
        m = _SIG_README.match(sq[0]) or _SIG_CANON.match(sq[0])
        if m and m.group(3) in by_name:
            if by_name[m.group(3)].dtype not in ("float16", "float32"):
                raise NotImplementedError("sigmoid: float16 or float32 only")
            return OpMatch("sigmoid", op_name, specs, m.group(1), dict(x=m.group(3), dtype=by_name[m.group(3)].dtype))
    raise NotImplementedError(
        "this IR is outside the hand-written operator family (W4A16 dequant-matmul, sigmoid, row softmax); "
        "antares_b200 has no general code generator and no fallback:\n  " + "\n  ".join(stmts))

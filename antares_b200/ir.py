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
    kind: str                       # "w4a16" | "sigmoid" | "softmax" | "eltwise"
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
    if len(stmts) >= 2:
        # reduce + map chains: compiled, then either recognised as row softmax by structure (hand-written
        # kernel) or run on the row-reduction template
        try:
            rp = compile_row_program(stmts, [s.name for s in specs])
        except NotImplementedError as e:
            row_reason = str(e)
        else:
            bad = [n for n in rp["mats"] + rp["cols"] if by_name[n].dtype not in ("float16", "float32")]
            if bad:
                row_reason = "row program: %s must be float16 or float32" % ", ".join(bad)
            elif any(len(by_name[n].dims) != len(rp["axes"]) for n in rp["mats"]) or any(len(by_name[n].dims) != 1 for n in rp["cols"]):
                row_reason = "row program: operand ranks do not match their indices"
            elif is_softmax_program(rp) and len(rp["axes"]) == 2:
                x = rp["mats"][0]
                return OpMatch("softmax", name or rp["out"], specs, rp["out"], dict(x=x, dtype=by_name[x].dtype))
            else:
                return OpMatch("rowprog", name or rp["out"], specs, rp["out"], rp)
    if len(sq) == 1:
        m = _SIG_README.match(sq[0]) or _SIG_CANON.match(sq[0])
        if m and m.group(3) in by_name:
            if by_name[m.group(3)].dtype not in ("float16", "float32"):
                raise NotImplementedError("sigmoid: float16 or float32 only")
            return OpMatch("sigmoid", op_name, specs, m.group(1), dict(x=m.group(3), dtype=by_name[m.group(3)].dtype))
    if len(stmts) == 1:
        # any other single element-wise statement: the interpreter kernel
        try:
            out_name, axes, used, prog, consts = compile_elementwise(stmts[0], [s.name for s in specs])
        except NotImplementedError as e:
            reason = str(e)
        else:
            bad = [n for n in used if by_name[n].dtype not in ("float16", "float32")]
            if not bad and all(len(by_name[n].dims) == len(axes) for n in used):
                return OpMatch("eltwise", name or out_name, specs, out_name, dict(inputs=used, program=prog, consts=consts, axes=axes))
            reason = "element-wise IR: inputs must be float16/float32 tensors of the output's rank"
    else:
        reason = row_reason if len(stmts) >= 2 else "empty program"
    raise NotImplementedError(
        "this IR is outside the operator family (W4A16 dequant-matmul, sigmoid, row softmax, single element-wise statements, "
        "row-reduction chains closed by one map statement); "
        "antares_b200 has no general code generator and no fallback (%s):\n  " % reason + "\n  ".join(stmts))


# ---- general element-wise statements -------------------------------------------------------------------
# `out[A, B] = expr` where every tensor in expr is indexed by exactly the output's axis list.  The
# expression is compiled to a small stack program that one CUDA kernel interprets (csrc/eltwise_vm.cu):
# the generic route for fusions outside the named operator family (lang/einstein_v2.py:297-578 is the
# reference's general front end; this covers its element-wise subset: + - * /, unary minus, numeric
# constants, .call(`f`) / .call(strs.f) with the functions below, .call(`max`|`min`|`pow`, [expr]),
# and dtype casts, which are no-ops here because the interpreter computes in fp32).

VM_OPS = {"in": 0, "const": 1, "add": 2, "sub": 3, "mul": 4, "div": 5, "neg": 6, "exp": 7, "log": 8, "sqrt": 9, "rsqrt": 10,
          "tanh": 11, "erf": 12, "sin": 13, "cos": 14, "abs": 15, "floor": 16, "ceil": 17, "max": 18, "min": 19, "pow": 20,
          "sigmoid": 21, "row": 22, "col": 23, "collen": 24}
_VM_UNARY = ("exp", "log", "sqrt", "rsqrt", "tanh", "erf", "sin", "cos", "abs", "floor", "ceil", "sigmoid")
_VM_BINARY_CALL = ("max", "min", "pow")
VM_MAX_OPS, VM_MAX_CONSTS, VM_MAX_INPUTS, VM_MAX_STACK = 48, 16, 8, 8

_TOKEN = re.compile(r"\s*(?:(\d+\.\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?|\d+(?:[eE][-+]?\d+)?)|([A-Za-z_]\w*)|(`[^`]*`)|(.))")


def _tokenise(text):
    out, pos = [], 0
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m:
            break
        pos = m.end()
        num, ident, quoted, sym = m.groups()
        if num is not None:
            out.append(("num", num))
        elif ident is not None:
            out.append(("id", ident))
        elif quoted is not None:
            out.append(("str", quoted[1:-1]))
        elif sym and not sym.isspace():
            out.append(("sym", sym))
    return out


class _EltParser:
    def __init__(self, tokens, axes, input_names, temps=None, cols=None):
        self.t, self.i, self.axes, self.names = tokens, 0, axes, input_names
        self.prog, self.consts, self.used = [], [], []
        self.depth = self.max_depth = 0
        # row programs only: results of earlier reduction statements (name -> stage), [cols] vectors seen so far
        self.temps, self.cols = temps, cols

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else ("end", "")

    def take(self, kind=None, val=None):
        k, v = self.peek()
        if (kind and k != kind) or (val is not None and v != val):
            raise NotImplementedError("element-wise IR: expected %s %r, found %r" % (kind or "", val or "", v))
        self.i += 1
        return v

    def emit(self, op, arg=0, delta=0):
        self.prog.append((VM_OPS[op], arg))
        self.depth += delta
        self.max_depth = max(self.max_depth, self.depth)

    def expr(self):
        self.term()
        while self.peek() in (("sym", "+"), ("sym", "-")):
            op = self.take()
            self.term()
            self.emit("add" if op == "+" else "sub", delta=-1)

    def term(self):
        self.unary()
        while self.peek() in (("sym", "*"), ("sym", "/")):
            op = self.take()
            self.unary()
            self.emit("mul" if op == "*" else "div", delta=-1)

    def unary(self):
        if self.peek() == ("sym", "-"):
            self.take()
            self.unary()
            self.emit("neg")
        else:
            self.postfix()

    def postfix(self):
        self.primary()
        while self.peek() == ("sym", "."):
            self.take()
            method = self.take("id")
            self.take("sym", "(")
            if method == "call":
                fname = self.func_name()
                if self.peek() == ("sym", ","):
                    self.take()
                    self.take("sym", "[")
                    self.expr()
                    self.take("sym", "]")
                    if fname not in _VM_BINARY_CALL:
                        raise NotImplementedError("element-wise IR: %s takes no second operand" % fname)
                    self.emit(fname, delta=-1)
                elif fname in _VM_UNARY:
                    self.emit(fname)
                else:
                    raise NotImplementedError("element-wise IR: function %r is not supported" % fname)
                self.take("sym", ")")
            elif method in ("cast", "to", "like"):  # dtype changes: the interpreter computes in fp32
                depth = 1
                while depth:
                    k, v = self.peek()
                    if k == "end":
                        raise NotImplementedError("element-wise IR: unbalanced parentheses")
                    self.i += 1
                    depth += (v == "(") - (v == ")") if k == "sym" else 0
            else:
                raise NotImplementedError("element-wise IR: method .%s() is not supported" % method)

    def func_name(self):
        k, v = self.peek()
        if k == "str":
            self.take()
            return v
        if k == "id" and v == "strs":
            self.take()
            self.take("sym", ".")
            return self.take("id")
        raise NotImplementedError("element-wise IR: .call() needs `name` or strs.name")

    def primary(self):
        k, v = self.peek()
        if k == "num":
            self.take()
            self.const(float(v))
        elif k == "sym" and v == "(":
            self.take()
            self.expr()
            self.take("sym", ")")
        elif k == "id" and v == "const":
            self.take()
            self.take("sym", "(")
            neg = self.peek() == ("sym", "-")
            if neg:
                self.take()
            self.const((-1 if neg else 1) * float(self.take("num")))
            self.take("sym", ")")
        elif k == "id" and self.temps is not None and v == self.axes[-1] and self.t[self.i + 1:self.i + 5] == [("sym", "."), ("id", "val"), ("sym", "("), ("sym", ")")]:
            self.i += 5                      # C.val(): the extent of the reduced axis
            self.emit("collen", 0, delta=1)
        elif k == "id":
            self.take()
            if v not in self.names and not (self.temps is not None and v in self.temps):
                raise NotImplementedError("element-wise IR: %r is not a declared input" % v)
            self.take("sym", "[")
            idx = []
            while self.peek() != ("sym", "]"):
                kk, vv = self.peek()
                self.take()
                if kk == "id":
                    idx.append(vv)
                elif not (kk == "sym" and vv == ","):
                    raise NotImplementedError("element-wise IR: only plain axis indices are supported")
            self.take("sym", "]")
            if self.temps is not None and v in self.temps:
                if idx != self.axes[:-1]:
                    raise NotImplementedError("row program: %s is a row result and must be indexed by %s" % (v, self.axes[:-1]))
                self.emit("row", self.temps[v], delta=1)
            elif self.temps is not None and idx == self.axes[-1:] and len(self.axes) > 1:
                if v not in self.cols:
                    self.cols.append(v)
                self.emit("col", self.cols.index(v), delta=1)
            else:
                if idx != self.axes:
                    raise NotImplementedError("element-wise IR: %s is indexed by %s, the output by %s" % (v, idx, self.axes))
                if v not in self.used:
                    self.used.append(v)
                self.emit("in", self.used.index(v), delta=1)
        else:
            raise NotImplementedError("element-wise IR: unexpected %r" % v)

    def const(self, c):
        if c not in self.consts:
            self.consts.append(c)
        self.emit("const", self.consts.index(c), delta=1)


def compile_elementwise(stmt, input_names):
    """'out[N] = expr' -> (output name, axes, input names in stack-program order, program, constants).
    Raises NotImplementedError when the statement is not purely element-wise."""
    m = re.match(r"^\s*([a-z_]\w*)\s*\[([^\]]*)\]\s*=(?!=)(.*)$", stmt, re.S)
    if not m:
        raise NotImplementedError("element-wise IR: not an assignment: %r" % stmt)
    out_name, axes_text, rhs = m.groups()
    axes = [a.strip() for a in axes_text.split(",") if a.strip()]
    if not axes or not all(re.fullmatch(r"[A-Z]\w*", a) for a in axes):
        raise NotImplementedError("element-wise IR: the output must be indexed by plain axes")
    p = _EltParser(_tokenise(rhs), axes, list(input_names))
    p.expr()
    if p.peek()[0] != "end":
        raise NotImplementedError("element-wise IR: trailing text %r" % (p.peek()[1],))
    if len(p.prog) > VM_MAX_OPS or len(p.consts) > VM_MAX_CONSTS or len(p.used) > VM_MAX_INPUTS or p.max_depth > VM_MAX_STACK:
        raise NotImplementedError("element-wise IR: expression too large for the interpreter (%d ops, %d constants, %d inputs, depth %d)"
                                  % (len(p.prog), len(p.consts), len(p.used), p.max_depth))
    if not p.used:
        raise NotImplementedError("element-wise IR: the expression reads no input tensor")
    return out_name, axes, p.used, p.prog, p.consts


# ---- reduce + map statement chains over one [rows..., cols] index space ------------------------------------
# `t0[N] >=! f0(x[N, C]); t1[N] +=! f1(x[N, C], t0[N]); out[N, C] = g(x[N, C], t0[N], t1[N], w[C], C.val())`:
# the softmax and layernorm forms of AntaresIR.md:226,232.  Every statement's expression becomes a stack
# program; one kernel (csrc/rowreduce_vm.cu) runs all stages of a row back to back.

ROW_MAX_STAGES, ROW_MAX_MAT, ROW_MAX_COL = 4, 4, 4
_REDUCE_KIND = {"+": 1, ">": 2, "<": 3}


def compile_row_program(stmts, input_names):
    """Statements -> dict(out, axes, stages=[(kind, program)], consts, mats, cols) with kind 0 map / 1 sum /
    2 max / 3 min; `mats` are the [axes] inputs and `cols` the [last axis] inputs in operand order.
    Raises NotImplementedError when the program is not a chain of row reductions closed by one map."""
    if not 2 <= len(stmts) <= ROW_MAX_STAGES:
        raise NotImplementedError("row program: 2..%d statements" % ROW_MAX_STAGES)
    m = re.match(r"^\s*([a-z_]\w*)\s*\[([^\]]*)\]\s*=(?!=)(.*)$", stmts[-1], re.S)
    if not m:
        raise NotImplementedError("row program: the last statement must be a plain assignment")
    out_name, axes_text, rhs_last = m.groups()
    axes = [a.strip() for a in axes_text.split(",") if a.strip()]
    if len(axes) < 2 or not all(re.fullmatch(r"[A-Z]\w*", a) for a in axes):
        raise NotImplementedError("row program: the output must be indexed by two or more plain axes")
    temps, mats, cols, consts, stages = {}, [], [], [], []
    depth = 0

    def run(rhs, what):
        nonlocal depth
        p = _EltParser(_tokenise(rhs), axes, list(input_names), temps=dict(temps), cols=cols)
        p.used, p.consts = mats, consts      # operand tables are shared by all stages
        p.expr()
        if p.peek()[0] != "end":
            raise NotImplementedError("row program: trailing text %r in %s" % (p.peek()[1], what))
        if len(p.prog) > VM_MAX_OPS:
            raise NotImplementedError("row program: %s is too long for the interpreter (%d operations)" % (what, len(p.prog)))
        depth = max(depth, p.max_depth)
        return p.prog

    for i, stmt in enumerate(stmts[:-1]):
        r = re.match(r"^\s*([a-z_]\w*)\s*\[([^\]]*)\]\s*([+<>])=!?(.*)$", stmt, re.S)
        if not r:
            raise NotImplementedError("row program: statement %d is not a +=, >= or <= reduction" % (i + 1))
        name, idx_text, op, rhs = r.groups()
        idx = [a.strip() for a in idx_text.split(",") if a.strip()]
        if idx != axes[:-1]:
            raise NotImplementedError("row program: %s must be indexed by %s (the output's axes without the reduced one)" % (name, axes[:-1]))
        stages.append((_REDUCE_KIND[op], run(rhs, "statement %d" % (i + 1))))
        temps[name] = i
    stages.append((0, run(rhs_last, "the last statement")))
    if not mats:
        raise NotImplementedError("row program: no [%s] input is read" % ", ".join(axes))
    if len(mats) > ROW_MAX_MAT or len(cols) > ROW_MAX_COL or len(consts) > VM_MAX_CONSTS or depth > VM_MAX_STACK:
        raise NotImplementedError("row program: too many operands for the interpreter")
    return dict(out=out_name, axes=axes, stages=stages, consts=consts, mats=mats, cols=cols)


def is_softmax_program(rp):
    """True when a compiled row program is row softmax whatever its tensors are called and however the text
    is spaced or parenthesised: max of x; sum of exp(x - max); exp(x - max) / sum."""
    o = VM_OPS
    sub_exp = [(o["in"], 0), (o["row"], 0), (o["sub"], 0), (o["exp"], 0)]
    want = [(2, [(o["in"], 0)]), (1, sub_exp), (0, sub_exp + [(o["row"], 1), (o["div"], 0)])]
    return len(rp["mats"]) == 1 and not rp["cols"] and [(k, list(pr)) for k, pr in rp["stages"]] == want

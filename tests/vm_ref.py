"""numpy evaluation of the interpreter programs that antares_b200.ir compiles (test helper)."""
from antares_b200.ir import VM_OPS


def eval_program_numpy(prog, consts, arrays, rows=None, cols=None, ncols=None):
    """Reference evaluation of a stack program (numpy, fp32): `arrays` are the element-wise / [rows, cols]
    inputs, `rows` the [rows, 1] results of earlier reduction stages, `cols` the [cols] vectors."""
    import numpy as np
    from math import erf as _erf
    inv = {v: k for k, v in VM_OPS.items()}
    st = []
    f32 = np.float32
    for op, arg in prog:
        name = inv[op]
        if name == "in":
            st.append(np.asarray(arrays[arg], dtype=f32))
        elif name == "const":
            st.append(f32(consts[arg]))
        elif name == "row":
            st.append(np.asarray(rows[arg], dtype=f32))
        elif name == "col":
            st.append(np.asarray(cols[arg], dtype=f32)[None, :])
        elif name == "collen":
            st.append(f32(ncols))
        elif name in ("add", "sub", "mul", "div", "max", "min", "pow"):
            b, a = st.pop(), st.pop()
            st.append({"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide, "max": np.maximum, "min": np.minimum,
                       "pow": np.power}[name](a, b).astype(f32))
        else:
            a = st.pop()
            fn = {"neg": np.negative, "exp": np.exp, "log": np.log, "sqrt": np.sqrt, "rsqrt": lambda v: 1 / np.sqrt(v), "tanh": np.tanh,
                  "erf": np.vectorize(_erf, otypes=[f32]), "sin": np.sin, "cos": np.cos, "abs": np.abs, "floor": np.floor, "ceil": np.ceil,
                  "sigmoid": lambda v: 1 / (1 + np.exp(-v))}[name]
            st.append(np.asarray(fn(a), dtype=f32))
    assert len(st) == 1
    return st[0]


def eval_row_program_numpy(rp, mats, cols):
    """Runs a compiled row program (ir.compile_row_program) on [rows, cols] numpy arrays."""
    import numpy as np
    rows_out = []
    ncols = mats[0].shape[-1]
    for kind, prog in rp["stages"]:
        v = np.broadcast_to(eval_program_numpy(prog, rp["consts"], mats, rows_out, cols, ncols), mats[0].shape)
        if kind == 0:
            return v.astype(np.float32)
        red = {1: np.sum, 2: np.max, 3: np.min}[kind](v.astype(np.float32), axis=-1, keepdims=True)
        rows_out.append(red.astype(np.float32))


"""Build recipe for the CPU oracle (test infrastructure, never shipped or benchmarked as product).

  python -m oracle.build            # builds both targets below

1. oracle/libantares_oracle.so  <- oracle/antares_oracle.c   (our plain-C restatement)
2. oracle/_ref/libantares_ref_mcpu.so <- oracle/ref_shim.cpp compiled against the reference's
   own headers where they lie in the reference checkout (graph_evaluator/execute_module.hpp,
   backends/c-mcpu/include/backend.hpp); compile flags follow graph_evaluator/client.py:52-57.
   Only built when the reference checkout is present; the built file is what travels.
3. oracle/_ref/evaluator.c-mcpu and oracle/_ref/evaluator.c-b200 <- the reference's unmodified
   graph_evaluator/run_graph.cpp, once against its own CPU HAL (backends/c-mcpu/include) and once
   against this repository's HAL for the B200 kernel library (include/c-b200/backend.hpp, linked
   with antares_b200/libantares_b200.so): the same evaluator prints `- K/i:` digests and `- TPR:`
   for both, which is how the reference cross-checks backends (antares/antares_compiler.py:506-520).
   Compile line after graph_evaluator/client.py:52-65.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: ANTARES_REFERENCE_ROOT, or a `reference` directory beside the repository
REFERENCE_ROOT = os.environ.get("ANTARES_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

ORACLE_SO = os.path.join(HERE, "libantares_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libantares_ref_mcpu.so")


def _newer(target, *sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "antares_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cmd = ["gcc", "-O3", "-ffp-contract=off", "-mavx2", "-mf16c", "-fopenmp", "-fPIC", "-shared",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(force=False):
    """Returns the path of the reference-runtime library, or None if it cannot be built here."""
    src = os.path.join(HERE, "ref_shim.cpp")
    inc_eval = os.path.join(REFERENCE_ROOT, "graph_evaluator")
    inc_backend = os.path.join(REFERENCE_ROOT, "backends", "c-mcpu", "include")
    if not os.path.isdir(inc_eval) or not os.path.isdir(inc_backend):
        return REF_SO if os.path.exists(REF_SO) else None
    deps = [src, os.path.join(inc_eval, "execute_module.hpp"), os.path.join(inc_backend, "backend.hpp")]
    if not force and _newer(REF_SO, *deps):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", src, "-o", REF_SO, "-shared", "-fPIC", "-O2",
           '-D__BACKEND__="c-mcpu"', "-D__BACKEND_mcpu__", "-std=c++17",
           "-Wno-string-compare", "-Wno-unused-result", "-Wno-unused-value",
           "-I" + inc_eval, "-I" + inc_backend, "-ldl", "-lpthread"]
    subprocess.check_call(cmd)
    return REF_SO


EVAL_MCPU = os.path.join(REF_DIR, "evaluator.c-mcpu")
EVAL_B200 = os.path.join(REF_DIR, "evaluator.c-b200")


def build_evaluators(force=False):
    """The reference's evaluator executable for its CPU backend and for the c-b200 HAL.  Returns the two
    paths (None where one cannot be built here: no reference checkout, or the kernel library not built)."""
    repo = os.path.dirname(HERE)
    src = os.path.join(REFERENCE_ROOT, "graph_evaluator", "run_graph.cpp")
    lib_dir = os.path.join(repo, "antares_b200")
    hal = os.path.join(repo, "include", "c-b200", "backend.hpp")
    out = []
    have_src = os.path.exists(src)
    common = ["-std=c++17", "-O2", "-Wno-string-compare", "-Wno-unused-result", "-Wno-unused-value", "-Wno-format"]
    targets = ((EVAL_MCPU, ['-D__BACKEND__="c-mcpu"', "-D__BACKEND_mcpu__", "-I" + os.path.join(REFERENCE_ROOT, "backends", "c-mcpu", "include")],
                ["-ldl", "-lpthread"], [os.path.join(REFERENCE_ROOT, "backends", "c-mcpu", "include", "backend.hpp")]),
               (EVAL_B200, ['-D__BACKEND__="c-b200"', "-I" + os.path.join(repo, "include", "c-b200"), "-I" + os.path.join(repo, "include")],
                ["-L" + lib_dir, "-lantares_b200", "-Wl,-rpath,$ORIGIN/../../antares_b200", "-ldl", "-lpthread"],
                [hal, os.path.join(repo, "include", "antares_b200.h"), os.path.join(lib_dir, "libantares_b200.so")]))
    for target, defs, libs, deps in targets:
        if not have_src or not all(os.path.exists(d) for d in deps):
            out.append(target if os.path.exists(target) else None)
            continue
        if force or not _newer(target, src, *deps):
            os.makedirs(REF_DIR, exist_ok=True)
            subprocess.check_call(["g++", src, "-o", target] + common + defs + libs)
        out.append(target)
    return tuple(out)


def build_all(force=False):
    return build_oracle(force), build_ref(force), build_evaluators(force)


if __name__ == "__main__":
    o, r, ev = build_all(force="--force" in sys.argv)
    print("oracle:", o)
    print("reference runtime:", r if r else "not built (reference checkout absent)")
    print("reference evaluator (c-mcpu, c-b200):", ev)

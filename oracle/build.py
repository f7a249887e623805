"""Build recipe for the CPU oracle (test infrastructure, never shipped or benchmarked as product).

  python -m oracle.build            # builds both targets below

1. oracle/libantares_oracle.so  <- oracle/antares_oracle.c   (our plain-C restatement)
2. oracle/_ref/libantares_ref_mcpu.so <- oracle/ref_shim.cpp compiled against the reference's
   own headers where they lie in the reference checkout (graph_evaluator/execute_module.hpp,
   backends/c-mcpu/include/backend.hpp); compile flags follow graph_evaluator/client.py:52-57.
   Only built when the reference checkout is present; the built file is what travels.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("ANTARES_REFERENCE_ROOT", "/root/reference")

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


def build_all(force=False):
    return build_oracle(force), build_ref(force)


if __name__ == "__main__":
    o, r = build_all(force="--force" in sys.argv)
    print("oracle:", o)
    print("reference runtime:", r if r else "not built (reference checkout absent)")

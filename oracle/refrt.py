"""ctypes wrapper of oracle/_ref/libantares_ref_mcpu.so: the reference's own CPU runtime
(ExecutionModule + c-mcpu backend) running hand-restated kernel-source texts.

TEST INFRASTRUCTURE ONLY.  Used to pin the C oracle, to generate tests/golden/, and as the timed
"reference" CPU baseline of the benchmark.  Needs g++ at run time (the reference JIT-compiles the
kernel text when a module is created).
"""
import ctypes
import os
import tempfile

import numpy as np

from . import build as _build

_lib = None
_workdir = None


def available():
    return os.path.exists(_build.REF_SO) or _build.build_ref() is not None


def lib():
    global _lib, _workdir
    if _lib is None:
        path = _build.REF_SO if os.path.exists(_build.REF_SO) else _build.build_ref()
        if path is None:
            raise RuntimeError("reference runtime library is not built and the reference checkout is absent")
        L = ctypes.CDLL(path)
        L.ref_module_time.restype = ctypes.c_double
        _lib = L
        _workdir = tempfile.mkdtemp(prefix="antares_ref_")
    return _lib


def num_threads():
    return int(lib().ref_num_threads())


class RefModule:
    """One ExecutionModule.  Call with numpy arrays: inputs in `// GLOBALS` order, then outputs."""

    def __init__(self, source):
        L = lib()
        self.handle = L.ref_module_create(source.encode(), _workdir.encode())
        if self.handle < 0:
            raise RuntimeError("reference runtime rejected the kernel source (code %d)" % self.handle)
        self.n_in = L.ref_module_num_inputs(self.handle)
        self.n_out = L.ref_module_num_outputs(self.handle)

    def _argv(self, arrays):
        assert len(arrays) == self.n_in + self.n_out, (len(arrays), self.n_in, self.n_out)
        for a in arrays:
            assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"]
        return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])

    def __call__(self, *arrays):
        lib().ref_module_compute(self.handle, self._argv(arrays))

    def time(self, *arrays, max_runs=0):
        return float(lib().ref_module_time(self.handle, self._argv(arrays), int(max_runs)))

"""The C-ABI library loads without a GPU and exports every symbol include/antares_b200.h declares."""
import ctypes
import os
import re

from antares_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "antares_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ab200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert len(names) >= 15
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), "missing export %s" % n


def test_python_binding_covers_the_header():
    assert sorted(list(_lib.SIGNATURES) + _lib.OTHER_SYMBOLS) == _declared()


def test_python_signatures_have_the_headers_argument_counts():
    """A ctypes signature with one argument too few or too many corrupts the call silently: every entry of
    _lib.SIGNATURES must list as many arguments as the header's declaration of that function."""
    text = open(os.path.join(ROOT, "include", "antares_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    counts = {}
    for name, params in re.findall(r"\b(ab200_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        params = params.strip()
        counts[name] = 0 if params in ("", "void") else params.count(",") + 1
    for name, sig in _lib.SIGNATURES.items():
        assert name in counts, name
        assert len(sig) == counts[name], "%s: header declares %d arguments, the binding passes %d" % (name, counts[name], len(sig))


def test_abi_version_and_error_text_without_gpu():
    L = _lib.load()
    assert L.ab200_abi_version() == 1
    # argument validation happens before any CUDA call
    rc = L.ab200_w4a16_gemv(None, None, None, None, 1, 4096, 4096, 128, 0, None)
    assert rc == _lib.EINVAL and b"null" in L.ab200_last_error()
    rc = L.ab200_w4a16_gemv(16, 16, 16, 16, 17, 4096, 4096, 128, 0, None)
    assert rc == _lib.EINVAL and b"M=17" in L.ab200_last_error()
    rc = L.ab200_w4a16_gemv(16, 16, 16, 16, 1, 4100, 4096, 128, 0, None)
    assert rc == _lib.EINVAL

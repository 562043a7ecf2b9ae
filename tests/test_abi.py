"""The C-ABI library loads and exports exactly what include/cera_cuda.h declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cera_cuda.h")
LIB = os.path.join(ROOT, "cera_b200", "libcera_cuda.so")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cera_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    assert os.path.exists(LIB), "build the library first: python cera_b200/build.py"
    lib = ctypes.CDLL(LIB)
    names = _declared()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_python_binding_covers_the_header():
    from cera_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_header_has_no_cxx_or_torch_types():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    assert "std::" not in text and "torch" not in text and "at::" not in text
    assert 'extern "C"' in text


def test_last_error_is_callable_without_a_device():
    from cera_b200 import _lib
    assert isinstance(_lib.last_error(), str)

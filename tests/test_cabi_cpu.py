"""The C-ABI library loads without a GPU and exports every symbol the header declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from qvb8_b200 import build
    return build.build()


def _declared():
    names = []
    for h in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(qvb8r?_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_builds_and_exports_header_symbols(built):
    lib = ctypes.CDLL(built)
    declared = _declared()
    assert declared, "no declarations found in include/"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_binding_lists_the_same_symbols(built):
    from qvb8_b200 import lib
    assert sorted(lib.EXPORTS) == _declared()
    assert b"sm_100a" in lib.load().qvb8_version()


def test_host_side_argument_checks_need_no_gpu(built):
    from qvb8_b200 import lib
    L = lib.load()
    assert L.qvb8_decode(None, 0, None, None) == 1                       # QVB8_ERR_ARG: null pack
    assert b"null pack" in L.qvb8_last_error()
    assert L.qvb8_small_m_scratch_bytes(0, 128, 128) == 0                # out-of-range sizes need no scratch


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from qvb8_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        lib.load()

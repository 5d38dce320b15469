"""CPU tests of the drop-in boundary: the shared library loads without a GPU, exports every symbol
include/b2lstm.h declares, and rejects malformed input through status codes (no exceptions cross
the C ABI, no compute happens here)."""
import ctypes as C
import os
import re

import pytest

import b2lstm
from b2lstm.lib import SIGNATURES

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "b2lstm.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(b2lstm.library_path())
    names = declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), "libb2lstm.so does not export " + n


def test_python_binding_covers_the_header():
    assert sorted(SIGNATURES) == declared_functions()


def test_version_and_weight_count_need_no_gpu():
    assert b"sm_100a" in b2lstm.lib().b2_version()
    assert b2lstm.lstm_num_weights(512, 256, True) == 657152
    assert b2lstm.lstm_num_weights(64, 128, False) == 99200


def test_malformed_network_is_rejected_with_a_status():
    h = C.c_void_p()
    rc = b2lstm.lib().b2_net_create(b'{"layers": [', 4, 10, 1, C.byref(h))
    assert rc == -5 and not h
    assert b"json" in b2lstm.lib().b2_last_error_string()
    rc = b2lstm.lib().b2_net_create(b'{"layers":[{"type":"lstm","size":4},{"type":"sse","size":4}]}', 4, 10, 1, C.byref(h))
    assert rc == -5 and b"input" in b2lstm.lib().b2_last_error_string()


def test_both_transposes_rejected_like_the_reference():
    # helpers/Matrix.cu of the reference throws for (transposeA && transposeB); the C ABI returns BAD_ARG
    rc = b2lstm.lib().b2_matrix_multiply(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, None)
    assert rc == -5


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import sys
    L = sys.modules["b2lstm.lib"]
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "library_path", lambda: str(tmp_path / "libb2lstm.so"))
    with pytest.raises(b2lstm.B2Error):
        L.lib()

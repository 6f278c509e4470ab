"""The C-ABI library loads without a GPU and exports every symbol the header declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "functs_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(functs_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from functs_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/functs_b200.h but not exported: {missing}"
    # the ctypes table binds exactly the declared entry points
    assert sorted(_lib.SIGNATURES) == names


def test_argument_errors_without_gpu():
    from functs_b200 import _lib
    lib = _lib.lib
    assert lib.functs_b200_abi_version() == 2
    # invalid arguments are rejected on the host before any CUDA call
    rc = lib.functs_b200_rows_select_add_select_rev(None, None, 4, 4, 1, 1.0, None)
    assert rc == -1 and "null" in _lib.last_error()
    rc = lib.functs_b200_select_topk(1, 1, 10, 1, 5000, 1, 1, None)
    assert rc == -1 and "topk" in _lib.last_error()
    assert lib.functs_b200_group_lookup(b"no such group") == -4
    n = lib.functs_b200_group_count()
    assert n >= 8
    for i in range(n):
        sig = lib.functs_b200_group_signature(i)
        assert lib.functs_b200_group_lookup(sig) == i
    assert lib.functs_b200_yolo_scratch_bytes(64, 13, 26, 52, 10647 * 80, 1000) > 64 * 10647 * 80 * 8
    assert lib.functs_b200_lstm_scratch_bytes(64, 64, 512, 512) >= 64 * 64 * 2048 * 4

"""The C ABI library loads without a GPU, exports every function that
include/frnnt.h declares, and rejects bad arguments on the host (no launch)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from fast_rnnt_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "frnnt.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(frnnt_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 18, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_host_side_checks(lib):
    lib.frnnt_mi_lattice_bytes.restype = ctypes.c_size_t
    assert lib.frnnt_version() >= 100
    assert lib.frnnt_with_cuda() == 1
    # (S+T+1) diagonals of round_up(S+1, 32) floats per utterance + two edge vectors
    assert lib.frnnt_mi_lattice_bytes(0, 2, 100, 500) == 2 * (601 * 128 + 2 * (601 + 64)) * 4
    assert lib.frnnt_mi_rows_per_block(0) == 256 and lib.frnnt_mi_rows_per_block(1) == 128
    assert lib.frnnt_mi_lattice_bytes(7, 2, 100, 500) == 0          # bad dtype
    # argument errors are found before any CUDA call
    rc = lib.frnnt_mi_forward(ctypes.c_int(5), None, None, None, None, None, None, 1, 1, 1, 0, None)
    assert rc == -1 and b"dtype" in lib.frnnt_last_error()
    rc = lib.frnnt_mi_forward(ctypes.c_int(0), None, None, None, None, None, None, 1, 5000, 10, 0, None)
    assert rc == -1 and b"ans is NULL" in lib.frnnt_last_error()
    rc = lib.frnnt_prune_ranges(ctypes.c_int(0), None, None, None, None, 1, 4, 4, 5, 9, None)
    assert rc == -1


def test_package_fails_loudly_without_the_library(monkeypatch, tmp_path):
    from fast_rnnt_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(_lib.FrnntError):
        _lib.lib()

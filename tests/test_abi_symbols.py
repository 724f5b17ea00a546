"""The C-ABI library loads and exports every symbol the public header declares (no GPU needed)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kfa.h")
LIB = os.path.join(ROOT, "kohakufa-cute_b200", "kohakufa_cute", "libkfa.so")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"KFA_API[^;(]*?\b(kfa_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("kfa_forward", "kfa_backward", "kfa_neighborhood_forward", "kfa_neighborhood_backward",
                     "kfa_center_keys", "kfa_merge_partial", "kfa_last_error"):
        assert required in names


@pytest.mark.skipif(not os.path.exists(LIB), reason="libkfa.so has not been built")
def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(LIB)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    lib.kfa_version.restype = ctypes.c_int
    assert lib.kfa_version() >= 1
    lib.kfa_last_error.restype = ctypes.c_char_p
    assert lib.kfa_last_error() == b""


@pytest.mark.skipif(not os.path.exists(LIB), reason="libkfa.so has not been built")
def test_python_binding_lists_every_declared_symbol():
    from kohakufa_cute import native

    assert sorted(native.SIGNATURES) == declared_symbols()
    native.library()


@pytest.mark.skipif(not os.path.exists(LIB), reason="libkfa.so has not been built")
def test_argument_errors_are_reported_without_a_gpu():
    from kohakufa_cute import native

    lib = native.library()
    record = native.KfaTensor()
    record.data = 16
    record.dtype = native.KFA_F32
    record.ndim = 4
    for i in range(4):
        record.sizes[i] = 2
        record.strides[i] = 1
    code = lib.kfa_forward(ctypes.byref(record), ctypes.byref(record), ctypes.byref(record), None, None, None, None,
                           None, 1.0, 0, None)
    assert code == 1
    assert b"FP16/BF16" in lib.kfa_last_error()

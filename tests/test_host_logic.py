"""Host-side logic of the CUDA library that needs no GPU: exported symbols, workspace sizing and the
error paths that are decided before any device call."""
import ctypes
import os
import re

import numpy as np
import pytest

from mkharness import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(product_lib_path):
    lib = ctypes.CDLL(product_lib_path)
    lib.mk_workspace_bytes.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p]
    lib.mk_workspace_bytes.restype = ctypes.c_size_t
    lib.cck_last_error.restype = ctypes.c_char_p
    lib.cck_mk_sample.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                  ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_int]
    return lib


@pytest.fixture(scope="module")
def tiny_sizes(make_case):
    x, meta = make_case(32, 1, 20, True)
    return (ctypes.c_size_t * 74)(*[a.nbytes for a in x]), meta


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "cck_b200.h")).read()
    names = re.findall(r"^\s*(?:const\s+)?[a-z_]+\s*\*?\s*((?:mk|cck)_[a-z_]+)\(", header, flags=re.M)
    assert {"cck_mk_sample", "mk_workspace_bytes", "mk_setup", "mk_run", "mk_read", "mk_gemm_test"} <= set(names)
    for name in names:
        getattr(lib, name)


def test_workspace_bytes(lib, tiny_sizes):
    sizes, meta = tiny_sizes
    total = lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, 0, sizes)
    # at least the pair-logit tables and the token modulations
    assert total >= 24 * 16 * 64 * 64 * 2 + 24 * 6 * 32 * 768 * 2
    assert total % 256 == 0
    more = lib.mk_workspace_bytes(2, meta["N"], meta["NS"], 20, 0, sizes)
    assert more > total


def test_workspace_bytes_rejects_inconsistent_sizes(lib, tiny_sizes):
    sizes, meta = tiny_sizes
    bad = (ctypes.c_size_t * 74)(*sizes)
    bad[synth.IN["WO"]] -= 2
    assert lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, 0, bad) == 0
    assert b"input" in lib.cck_last_error()
    # more steps than SIGMA holds
    assert lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 21, 0, sizes) == 0
    # a token count that does not match the buffers
    assert lib.mk_workspace_bytes(meta["S"], meta["N"] + 1, meta["NS"], 20, 0, sizes) == 0


def test_unsupported_flags_are_refused(lib, tiny_sizes):
    sizes, meta = tiny_sizes
    for bit in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512):
        assert lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, bit, sizes) == 0
        assert b"not built" in lib.cck_last_error()


def test_operator_errors_before_any_device_work(lib, tiny_sizes):
    sizes, meta = tiny_sizes
    ptrs = (ctypes.c_void_p * 74)()
    # wrong arity
    assert lib.cck_mk_sample(None, None, ptrs, sizes, 73, None, meta["N"], None, 0, 1, 20, 0) == 1
    assert lib.cck_last_error() == b"MkSample: wrong number of inputs"
    # workspace too small
    assert lib.cck_mk_sample(None, None, ptrs, sizes, 74, None, meta["N"], None, 1024, 1, 20, 0) == 2
    assert lib.cck_last_error() == b"MkSample: workspace too small"
    # a variant flag
    assert lib.cck_mk_sample(None, None, ptrs, sizes, 74, None, meta["N"], None, 1 << 40, 1, 20, 128) == 4
    # inconsistent sizes
    bad = (ctypes.c_size_t * 74)(*sizes)
    bad[synth.IN["ENC_W2"]] += 2
    assert lib.cck_mk_sample(None, None, ptrs, bad, 74, None, meta["N"], None, 1 << 40, 1, 20, 0) == 3

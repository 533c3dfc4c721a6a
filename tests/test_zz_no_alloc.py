"""The operator entry point that takes no workspace (cck_mk_sample_static).

Some callers of the sampler cannot allocate device memory: XLA runs the operator while it records a
command buffer (a CUDA graph) and a C caller may be inside a capture of its own, where cudaMalloc is
refused. For them the library holds a fixed 32 MiB scratch array on the device. This test calls that
entry point through the C ABI twice in a row and checks both results against the ordinary entry
point (cck_mk_sample with a caller-owned workspace): same kernel, same inputs, so the positions must
be identical, which is well inside the 2e-2 gate the parity tests use. It also checks that a fold
too large for the built-in scratch is refused with a clear message instead of being run.

This file is collected last on purpose, so that a run stopping at the first failure has already
been through every other test.
"""
import ctypes

import numpy as np
import pytest

from mkharness import driver, synth

pytestmark = pytest.mark.gpu

ARGS = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]


def test_static_workspace_entry_point_matches_the_ordinary_one(product_lib_path, make_case):
    import torch

    lib = ctypes.CDLL(product_lib_path)
    lib.cck_last_error.restype = ctypes.c_char_p
    lib.cck_static_workspace_bytes.restype = ctypes.c_size_t
    lib.mk_workspace_bytes.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p]
    lib.mk_workspace_bytes.restype = ctypes.c_size_t
    ordinary = lib.cck_mk_sample
    ordinary.argtypes = ARGS + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    static = lib.cck_mk_sample_static
    static.argtypes = ARGS + [ctypes.c_int, ctypes.c_int, ctypes.c_int]

    x, meta = make_case(32, 1, 20, True)
    steps, seed = 3, 21
    dev = [torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda() for a in x]
    ptrs = (ctypes.c_void_p * 74)(*[t.data_ptr() for t in dev])
    sizes = (ctypes.c_size_t * 74)(*[a.nbytes for a in x])
    ext = torch.tensor([meta["N"], meta["NS"], 1, seed, 0], dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    shape = (1, meta["N"], 24, 3)

    need = lib.mk_workspace_bytes(1, meta["N"], meta["NS"], steps, 0, sizes)
    assert 0 < need <= lib.cck_static_workspace_bytes() == 32 << 20
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.zeros(shape, dtype=torch.float32, device="cuda")
    rc = ordinary(stream, ext.data_ptr(), ptrs, sizes, 74, want.data_ptr(), meta["N"], ws.data_ptr(), need, 1, steps, 0)
    assert rc == 0, lib.cck_last_error()
    torch.cuda.synchronize()
    want = want.cpu().numpy()
    assert np.isfinite(want).all() and np.abs(want).max() > 1.0

    for call in range(2):  # the second call finds the array full of the first call's data
        got = torch.full(shape, float(call + 5), dtype=torch.float32, device="cuda")
        rc = static(stream, ext.data_ptr(), ptrs, sizes, 74, got.data_ptr(), meta["N"], 1, steps, 0)
        assert rc == 0, lib.cck_last_error()
        torch.cuda.synchronize()
        got = got.cpu().numpy()
        assert driver.max_rel_err(got, want) <= 2e-2
        assert (got == want).all(), "same kernel and inputs: the positions must be identical"

    # another seed really changes the result (the array is not serving stale output)
    ext2 = torch.tensor([meta["N"], meta["NS"], 1, seed + 1, 0], dtype=torch.int32, device="cuda")
    other = torch.zeros(shape, dtype=torch.float32, device="cuda")
    assert static(stream, ext2.data_ptr(), ptrs, sizes, 74, other.data_ptr(), meta["N"], 1, steps, 0) == 0
    torch.cuda.synchronize()
    assert (other.cpu().numpy() != want).any()

    # a fold beyond the built-in scratch is refused, not run: 64 samples of the same inputs
    big = lib.mk_workspace_bytes(64, meta["N"], meta["NS"], steps, 0, sizes)
    assert big > lib.cck_static_workspace_bytes()
    out64 = torch.zeros((64,) + shape[1:], dtype=torch.float32, device="cuda")
    rc = static(stream, ext.data_ptr(), ptrs, sizes, 74, out64.data_ptr(), meta["N"], 64, steps, 0)
    assert rc == 2
    msg = lib.cck_last_error().decode()
    assert "built-in scratch holds %d" % (32 << 20) in msg and str(big) in msg
    torch.cuda.synchronize()
    assert float(out64.abs().max()) == 0.0

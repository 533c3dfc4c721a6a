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
    # ESM (a reference variant) and bit 16 (set aside for a variant of this library's own): known, not built
    for bit in (256, 1 << 16):
        assert lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, bit, sizes) == 0
        assert b"not built" in lib.cck_last_error()
    # bits that belong to nobody
    for bit in (1 << 10, 1 << 24):
        assert lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, bit, sizes) == 0
        assert b"no variant uses" in lib.cck_last_error()
    # the Heun variant is built: it needs room for the first slope
    plain = lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, 0, sizes)
    heun = lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], 20, synth.F_HEUN, sizes)
    assert heun >= plain + meta["S"] * meta["N"] * 24 * 3 * 4


END_NONE, END_SUB, END_PHASE = 0, 1, 2


def program(lib, mode, nsteps, flags):
    buf = (ctypes.c_ubyte * (4 * 160))()
    n = lib.mk_program(mode, nsteps, flags, buf, 160)
    assert 0 < n <= 160
    return np.frombuffer(bytes(buf), dtype=np.uint8).reshape(-1, 4)[:n]


def test_phase_program(lib):
    """The schedule the kernel interprets: one denoiser call has the reference's 191 phases
    (1 init, 9 encoder, 1 aggregation, 7 x 24 token blocks, 3 glue, 9 decoder), the token block is a
    loop of 7 phases, and Heun calls the denoiser twice per step."""
    euler = program(lib, 0, 5, 0)
    heun = program(lib, 0, 5, synth.F_HEUN)
    once = program(lib, 1, 0, 0)
    fn_ret = int(euler[-1, 0])  # the function codes' order: BLOCK_NEXT, STEP_NEXT, CALL, RET, END
    fn_end, fn_call, fn_step_next, fn_block_next = fn_ret + 1, fn_ret - 1, fn_ret - 2, fn_ret - 3
    for prog, calls in ((euler, 1), (heun, 2), (once, 1)):
        assert int((prog[:, 0] == fn_call).sum()) == calls
        assert int((prog[:, 0] == fn_end).sum()) == 1 and int(prog[-1, 0]) == fn_ret
        end = int(np.argmax(prog[:, 0] == fn_end))
        sub = prog[end + 1:-1]
        assert all(int(c[1]) == end + 1 for c in prog[prog[:, 0] == fn_call]), "calls point at the subroutine"
        # the subroutine: a loop of 7 phase-ending operations closed by one BLOCK_NEXT
        loop_at = int(np.argmax(sub[:, 0] == fn_block_next))
        first = int(sub[loop_at, 1]) - (end + 1)
        body = sub[first:loop_at]
        assert len(body) == 7 and all((b[3] & 3) == END_PHASE for b in body) and all(b[2] == 255 for b in body)
        phases = int(((sub[:, 3] & 3) == END_PHASE).sum())
        assert phases - 7 + 7 * 24 == 191
    assert len(heun) == len(euler) + 2
    assert int((euler[:, 0] == fn_step_next).sum()) == 1 and int((once[:, 0] == fn_step_next).sum()) == 0


def test_flow_program(lib):
    """With the program writer's flow bit the token block has one barrier instead of seven, after the
    adaLN pass that opens it: QKVG, attention, WO, the transition's adaLN, W1, W2 and the next block's
    adaLN share a phase (units and rows wait for completion counters). The attention is bracketed by
    CTA-level syncs because it restages shared memory, and one more stands before W1, whose tiles
    fill the ring slots that WO's epilogue borrows. PARALLEL and QKNORM blocks stay on barriers."""
    PROG_FLOW = 1 << 30
    base = program(lib, 0, 5, 0)
    flow = program(lib, 0, 5, PROG_FLOW)
    fn_ret = int(base[-1, 0])
    fn_block_next, fn_cta_sync = fn_ret - 3, fn_ret - 4
    def body(prog):
        end = int(np.argmax(prog[:, 0] == fn_ret + 1))
        sub = prog[end + 1:-1]
        loop_at = int(np.argmax(sub[:, 0] == fn_block_next))
        return sub[int(sub[loop_at, 1]) - (end + 1):loop_at]
    b0, b1 = body(base), body(flow)
    assert int(((b0[:, 3] & 3) != 0).sum()) == 7 and int(((b1[:, 3] & 3) != 0).sum()) == 1
    assert int((b1[:, 0] == fn_cta_sync).sum()) == 3
    work = lambda b: [tuple(int(v) for v in o[:3]) for o in b if int(o[0]) != fn_cta_sync]
    assert work(b0) == work(b1), "the same operations in the same order"
    for flags in (synth.F_PARALLEL, synth.F_QKNORM):
        assert np.array_equal(program(lib, 0, 5, flags), program(lib, 0, 5, flags | PROG_FLOW))


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
    assert lib.cck_mk_sample(None, None, ptrs, sizes, 74, None, meta["N"], None, 1 << 40, 1, 20, 256) == 4
    # inconsistent sizes
    bad = (ctypes.c_size_t * 74)(*sizes)
    bad[synth.IN["ENC_W2"]] += 2
    assert lib.cck_mk_sample(None, None, ptrs, bad, 74, None, meta["N"], None, 1 << 40, 1, 20, 0) == 3

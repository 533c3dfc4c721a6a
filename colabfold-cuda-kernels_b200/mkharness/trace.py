"""Event trace of one CTA over the first phases of a launch, from a diagnostics build of the library.

    python colabfold-cuda-kernels_b200/build.py --diag CCK_TRACE=1 -o /tmp/libcck_trace.so   # CTA 0
    python -m mkharness.trace --lib /tmp/libcck_trace.so [--tokens 512] [--samples 5] [--from-cycle A --to-cycle B]

Prints the events of the traced CTA in time order, one column per role (schedule thread, TMA, MMA,
first worker thread, second attention pipeline), cycles from the first event. The build records the
first 2048 events of each role, which reaches into the token blocks of the first sampling step, and
every CTA's wait at each grid barrier (--barriers prints those: the CTA that waited least arrived last).
Run from colabfold-cuda-kernels_b200/ (or with it on PYTHONPATH).
"""
import argparse
import ctypes

import numpy as np

from . import driver, synth

ROLES, SLOTS, BARRIERS, CTAS = 7, 2048, 1024, 160
NAMES = {
    0x10: "att TMA pair logits", 0x12: "att TMA K|V", 0x20: "att MMA sees P", 0x22: "att MMA P.V issued",
    0x24: "att MMA Q.K ahead", 0x30: "att waits S", 0x32: "att got S", 0x34: "att bias+max done", 0x38: "att P handed over",
    0x3a: "att waits O", 0x3c: "att got O", 0x3e: "att item done", 0x40: "att O loaded", 0x42: "att TO store issued",
    0x44: "att item begins", 0x50: "gemm TMA begins", 0x52: "gemm TMA tile ready", 0x54: "gemm TMA tile asked",
    0x60: "gemm MMA begins", 0x62: "gemm MMA acc free", 0x64: "gemm MMA operands", 0x66: "gemm MMA tile issued",
    0x70: "gemm EPI begins", 0x72: "gemm EPI acc read", 0x74: "gemm EPI reported", 0x76: "gemm EPI done",
    0x80: "op begins", 0x82: "op ends", 0x84: "barrier reached", 0x86: "barrier passed",
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", required=True)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--nsteps", type=int, default=2)
    ap.add_argument("--from-cycle", type=int, default=0)
    ap.add_argument("--to-cycle", type=int, default=1 << 62)
    ap.add_argument("--barriers", action="store_true")
    ap.add_argument("--on-barriers", action="store_true", help="token blocks on grid barriers instead of completion counters")
    a = ap.parse_args()
    x, meta = synth.make_inputs(a.tokens, samples=a.samples, steps=200, seed=0)
    lib = driver.MkLib(a.lib)
    lib.setup(x, meta)
    lib.set_flow(not a.on_barriers)
    rec = np.zeros((ROLES, SLOTS), np.uint64)
    n = (ctypes.c_uint * ROLES)()
    for _ in range(2):  # the second launch is the warm one
        lib.run(mode=0, nsteps=a.nsteps, seed=1)
        lib.lib.mk_trace(ctypes.c_void_p(rec.ctypes.data), n)
    waits = np.zeros((BARRIERS, CTAS), np.uint32)
    lib.lib.mk_barrier_waits(ctypes.c_void_p(waits.ctypes.data))
    lib.teardown()
    if a.barriers:
        kind, cyc = (waits >> 24)[:, 0], (waits & 0xFFFFFF).astype(np.int64)
        print("barrier kind  least-wait (CTA)  median  most (CTA)   [cycles]")
        for i in range(BARRIERS):
            c = cyc[i, :148]
            if c.sum() == 0:
                break
            print("%5d %4d  %8d (%3d) %8d %8d (%3d)" % (i, kind[i], c.min(), c.argmin(), np.median(c), c.max(), c.argmax()))
        return
    ev = np.concatenate([rec[r, :min(n[r], SLOTS)] for r in range(ROLES)])
    t = (ev >> np.uint64(16)).astype(np.int64)
    code = ((ev >> np.uint64(8)) & np.uint64(255)).astype(int)
    val = (ev & np.uint64(255)).astype(int)
    order = np.argsort(t, kind="stable")
    t0 = t[order[0]]
    for i in order:
        dt, c = t[i] - t0, int(code[i])
        if dt < a.from_cycle or dt > a.to_cycle:
            continue
        second = c < 0x50 and (c & 1)
        base = c & ~1 if c < 0x50 else c
        col = 4 if second else {1: 1, 2: 2, 3: 3, 4: 3, 5: 1, 6: 2, 7: 3, 8: 0}.get(base >> 4, 0)
        print("%10d %s%-22s %3d" % (dt, " " * (24 * col), NAMES.get(base, hex(c)), val[i]))


if __name__ == "__main__":
    main()

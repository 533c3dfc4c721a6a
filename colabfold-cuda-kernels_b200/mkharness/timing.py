"""Per-phase-kind timing of one fold from the library's own record (no profiler): wall time from grid
barrier to grid barrier, sampled by CTA 0, summed per kind of phase.

    python -m mkharness.timing [--tokens 512] [--samples 5] [--nsteps 200] [--barriers]

--barriers: every operation of a token block ends at a grid barrier (the reference's schedule), which
splits the block's time by operation; the default runs the blocks on completion counters.
Run from colabfold-cuda-kernels_b200/ (or with it on PYTHONPATH).
"""
import argparse

from . import driver, synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--nsteps", type=int, default=200)
    ap.add_argument("--barriers", action="store_true")
    ap.add_argument("--lib", default=driver.PRODUCT_LIB)
    a = ap.parse_args()
    x, meta = synth.make_inputs(a.tokens, samples=a.samples, steps=max(a.nsteps, 1), seed=0)
    lib = driver.MkLib(a.lib)
    lib.setup(x, meta)
    lib.set_flow(not a.barriers)
    lib.run(mode=0, nsteps=min(a.nsteps, 5), seed=1)  # warm-up
    ms, kinds = lib.run(mode=0, nsteps=a.nsteps, seed=1, timing=True)
    flops = synth.flops_per_eval(meta["N"], meta["A"], a.samples)
    print("N_token=%d samples=%d nsteps=%d, token blocks on %s: fold %.2f ms, %.3f ms/step, %.0f evals/s, %.1f TFLOP/s algorithmic"
          % (a.tokens, a.samples, a.nsteps, "grid barriers" if a.barriers else "completion counters", ms, ms / a.nsteps,
             a.samples * a.nsteps / ms * 1e3, flops * a.samples * a.nsteps / ms / 1e9))
    total = sum(w for w, _ in kinds.values())
    print("| kind | total ms | share | phases | µs/phase |\n|---|---|---|---|---|")
    for k, (w, n) in sorted(kinds.items(), key=lambda kv: -kv[1][0]):
        if n:
            print("| %s | %.2f | %.1f%% | %d | %.2f |" % (k, w, 100 * w / total, n, 1e3 * w / n))
    lib.teardown()


if __name__ == "__main__":
    main()

"""Generates the golden fixtures of the sampler from the reference's own CUDA kernel.

Run on a GPU box (the reference kernel needs a GPU):
    python tests/golden/make_golden.py <output dir> [case ...]
It loads oracle/_ref/libref_sm100.so (the reference's diffusion.cu compiled unmodified for sm_100 by
oracle/Makefile), drives it through its ctypes API on seeded synthetic inputs, and stores the buffers
it produces at fixed points of its schedule. The fixtures pin the CPU oracle (tests/test_oracle.py)
and, through it, the CUDA path.
"""
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "colabfold-cuda-kernels_b200"))
from mkharness import driver, synth  # noqa: E402

# (name, tokens, samples, steps, tiny atoms layout, sampled steps)
CASES = [
    ("tiny", 32, 1, 20, True, 20),
    ("ragged", 48, 2, 8, False, 3),
]
# the Heun variant (flag 128): name, tokens, samples, steps, tiny layout, sampled steps, churn
HEUN_CASES = [
    ("heun", 32, 1, 8, True, 4, 0.5),
]
# variants of the denoiser itself (SCFINAL 64: affine LayerNorm of the conditioning before its two bf16
# views; IDSCALE 32: modulations from the conditioning itself, linear scale slots, eps 0.1; CHAIN_K 1: the
# atom keys' input normalised from the rounded queries' input): name, flags
VARIANT_CASES = [("scfinal", 64), ("idscale", 32), ("chaink", 1), ("qknorm", 4), ("parallel", 8), ("atob", 2), ("chiral", 16)]
VARIANT_STOPS = {
    "enc0_proj": (3, ["AKV"]),
    "encoder": (11, ["SCBF", "SCLN0", "SE", "SKIP"]),
    "tok0_adaln": (13, ["TX"]),
    "tok0": (19, ["ACT"]),
    "final": (0, ["OUT", "UPD"]),
}
# QKNORM (4: LayerNorm of q and k, tokens and atoms) adds a phase to every token block
QKNORM_STOPS = {
    "enc0_proj": (3, ["AQG", "AKV"]),
    "tok0_qkn": (15, ["QKVG"]),
    "final": (0, ["OUT", "UPD"]),
}


# PARALLEL (8: attention and transition both read the block input) has four phases per token block
PARALLEL_STOPS = {
    "enc0": (5, ["QA"]),
    "tok0_adaln": (13, ["TX", "TX2"]),
    "tok0_qkvg": (14, ["QKVG", "TC"]),
    "tok0_attn": (15, ["TO", "ACT"]),
    "tok0": (16, ["ACT"]),
    "final": (0, ["OUT", "UPD"]),
}


# ATOB (2: a third, multiplying part in every GLU unit of the token and atom transitions)
ATOB_STOPS = {
    "enc0": (5, ["QA"]),
    "tok0_glu": (18, ["TC"]),
    "tok0": (19, ["ACT"]),
    "final": (0, ["OUT", "UPD"]),
}


# CHIRAL (16: the gradient of the chirality restraints enters the atom features)
CHIRAL_STOPS = {
    "atom_init": (2, ["QA"]),
    "final": (0, ["OUT", "UPD"]),
}


def variant_stops(name):
    return {"qknorm": QKNORM_STOPS, "parallel": PARALLEL_STOPS, "atob": ATOB_STOPS, "chiral": CHIRAL_STOPS}.get(name, VARIANT_STOPS)


REALIGN_CASES = [
    ("realign", 48, 2, 8, False, 3),
]
# phases of one denoiser call in the reference's schedule, and of a sampling run up to the first call
DENOISE_PHASES, HEAD_PHASES = 1 + 9 + 1 + 7 * 24 + 3 + 9, 3
T_ONCE = 20.0
# phases of the reference schedule in mode 1: 1 pair build, 1 atom init, 9 encoder, 1 aggregation,
# 7 per token block, 3 glue, 9 decoder, 1 output
STOPS = {
    "atom_init": (2, ["QA", "NTV"]),
    "enc0_proj": (3, ["AQG", "AKV", "SCT"]),
    "enc0_attn": (4, ["AO", "SCH"]),
    "enc0": (5, ["QA", "SC"]),
    "encoder": (11, ["SKIP", "ABF", "SE", "SCBF", "SCLN0"]),
    "aggr": (12, ["ACT"]),
    "tok0_adaln": (13, ["TX"]),
    "tok0_qkvg": (14, ["QKVG"]),
    "tok0_attn": (15, ["TO"]),
    "tok0_wo": (16, ["ACT"]),
    "tok0_glu": (18, ["TC"]),
    "tok0": (19, ["ACT"]),
    "tok1": (26, ["ACT"]),
    "tokens": (12 + 7 * 24, ["ACT"]),
    "final": (0, ["OUT", "UPD", "TB", "ACT"]),
}


# a fold told by masks inside a larger bucket (synth.masked_bucket_case): name, sampled steps
MASKED_CASES = [("masked", 3)]
MASKED_STOPS = {
    "atom_init": (2, ["QA"]),
    "enc0_attn": (4, ["AO"]),
    "aggr": (12, ["ACT"]),
    "tok0_attn": (15, ["TO"]),
    "tok0": (19, ["ACT"]),
    "final": (0, ["OUT", "UPD"]),
}


def input_digest(x):
    d = 0
    for a in x:
        d = zlib.crc32(np.ascontiguousarray(a).view(np.uint8), d)
    return d


KEEP = 8192  # elements kept of a large buffer


def subset(n):
    """Indices of the elements a fixture keeps of an n-element buffer: all of a small one, a seeded
    sorted sample of a large one."""
    if n <= 2 * KEEP:
        return np.arange(n)
    return np.sort(np.random.default_rng(1234).choice(n, KEEP, replace=False))


def pack(name, arr):
    arr = np.asarray(arr).ravel()
    arr = arr[subset(arr.size)]
    if name in driver.BF16_BUFS:
        return synth.to_bf16(arr)
    return arr.astype(np.float32)


def main(out_dir, only=()):
    os.makedirs(out_dir, exist_ok=True)
    ref = driver.MkLib(driver.REFERENCE_LIB)
    # a fold told by masks alone inside a larger bucket, extra pair logits present
    for name, run_steps in MASKED_CASES:
        if only and name not in only:
            continue
        x, meta = synth.masked_bucket_case()
        ref.setup(x, meta)
        xn = synth.noisy_positions(meta, T_ONCE)
        out = {"digest": np.array([input_digest(x)], dtype=np.uint64), "t": np.array([T_ONCE], dtype=np.float32)}
        for tag, (stop, bufs) in MASKED_STOPS.items():
            ref.run(mode=1, dbg_stop=stop, xn=xn, t=T_ONCE)
            for b in bufs:
                out["%s.%s" % (tag, b)] = pack(b, ref.read(b))
        ref.run(mode=0, nsteps=run_steps, dbg_stop=3, seed=7)
        out["step1.XN"] = pack("XN", ref.read("XN"))
        ref.run(mode=0, nsteps=run_steps, seed=7)
        out["sample.POS"] = pack("POS", ref.read("POS"))
        out["sample.steps"] = np.array([run_steps], dtype=np.int32)
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **out)
        print("wrote", name)
    if only and not (set(only) - {m[0] for m in MASKED_CASES}):
        ref.teardown()
        return
    for name, n_tok, samples, steps, tiny, run_steps in CASES:
        x, meta = synth.make_inputs(n_tok, samples=samples, steps=steps, seed=0, tiny=tiny)
        ref.setup(x, meta)
        xn = synth.noisy_positions(meta, T_ONCE)
        out = {"digest": np.array([input_digest(x)], dtype=np.uint64), "t": np.array([T_ONCE], dtype=np.float32)}
        for tag, (stop, bufs) in STOPS.items():
            ref.run(mode=1, dbg_stop=stop, xn=xn, t=T_ONCE)
            for b in bufs:
                out["%s.%s" % (tag, b)] = pack(b, ref.read(b))
        # sampling: the first step's noisy positions, and the trajectory's end
        ref.run(mode=0, nsteps=run_steps, dbg_stop=3, seed=7)
        out["step1.POS"] = pack("POS", ref.read("POS"))
        out["step1.XN"] = pack("XN", ref.read("XN"))
        ref.run(mode=0, nsteps=run_steps, seed=7)
        out["sample.POS"] = pack("POS", ref.read("POS"))
        out["sample.steps"] = np.array([run_steps], dtype=np.int32)
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **out)
        print("wrote", name, {k: v.shape for k, v in out.items() if k.endswith("OUT")})
    # Heun: the first half step (x1 in XN, the slope in GRAD), the first full step, the trajectory's end
    for name, n_tok, samples, steps, tiny, run_steps, churn in HEUN_CASES:
        x, meta = synth.make_inputs(n_tok, samples=samples, steps=steps, seed=0, tiny=tiny, flags=synth.F_HEUN, churn=churn)
        ref.setup(x, meta)
        out = {"digest": np.array([input_digest(x)], dtype=np.uint64), "churn": np.array([churn], dtype=np.float32)}
        half = HEAD_PHASES + DENOISE_PHASES + 1
        ref.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
        out["heun1.XN"] = pack("XN", ref.read("XN"))
        out["heun1.GRAD"] = pack("GRAD", ref.read("GRAD"))
        ref.run(mode=0, nsteps=run_steps, dbg_stop=half + DENOISE_PHASES + 1, seed=7)
        out["step1.POS"] = pack("POS", ref.read("POS"))
        ref.run(mode=0, nsteps=run_steps, seed=7)
        out["sample.POS"] = pack("POS", ref.read("POS"))
        out["sample.steps"] = np.array([run_steps], dtype=np.int32)
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **out)
        print("wrote", name)
    # REALIGN (512): the denoised positions and the alignment's moments, the aligned Euler step, a trajectory
    for name, n_tok, samples, steps, tiny, run_steps in REALIGN_CASES:
        x, meta = synth.make_inputs(n_tok, samples=samples, steps=steps, seed=0, tiny=tiny, flags=synth.F_REALIGN)
        ref.setup(x, meta)
        out = {"digest": np.array([input_digest(x)], dtype=np.uint64)}
        half = HEAD_PHASES + DENOISE_PHASES + 1
        ref.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
        out["moments.GRAD"] = pack("GRAD", ref.read("GRAD"))
        out["moments.KAB"] = pack("KAB", ref.read("KAB"))
        ref.run(mode=0, nsteps=run_steps, dbg_stop=half + 1, seed=7)
        out["step1.POS"] = pack("POS", ref.read("POS"))
        ref.run(mode=0, nsteps=run_steps, seed=7)
        out["sample.POS"] = pack("POS", ref.read("POS"))
        out["sample.steps"] = np.array([run_steps], dtype=np.int32)
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **out)
        print("wrote", name)
    # one denoiser call of each variant on the tiny layout
    for name, flags in VARIANT_CASES:
        x, meta = synth.make_inputs(32, samples=1, steps=20, seed=0, tiny=True, flags=flags)
        ref.setup(x, meta)
        xn = synth.noisy_positions(meta, T_ONCE)
        out = {"digest": np.array([input_digest(x)], dtype=np.uint64), "flags": np.array([flags], dtype=np.int32)}
        for tag, (stop, bufs) in variant_stops(name).items():
            ref.run(mode=1, dbg_stop=stop, xn=xn, t=T_ONCE)
            for b in bufs:
                out["%s.%s" % (tag, b)] = pack(b, ref.read(b))
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **out)
        print("wrote", name)
    ref.teardown()


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <output dir> [case ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))

"""The CPU oracle against the golden fixtures dumped from the reference's own CUDA kernel
(tests/golden/make_golden.py). This is the pin of the oracle: every checkpoint of one denoiser
evaluation, the first sampling step (all three Philox streams) and a short trajectory.

The reference computes in bf16 with f32 accumulation and fast device transcendentals; the oracle
rounds at the same points with libm functions, so buffers agree to bf16 resolution, and f32 buffers
that involve no bf16 product agree to f32 resolution.
"""
import os
import sys

import numpy as np
import pytest

from mkharness import driver, synth

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden as mg  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BF16_TOL = 1e-2   # max |a-b| / max |b| across a buffer that went through bf16 products
EXACT_TOL = 2e-6  # f32 buffers with no bf16 product on their path


def load(name):
    g = np.load(os.path.join(GOLDEN, "ref_%s.npz" % name))
    return {k: (synth.from_bf16(g[k]) if g[k].dtype == np.uint16 else g[k]) for k in g.files}


def picked(arr):
    arr = np.asarray(arr).ravel()
    return arr[mg.subset(arr.size)]


@pytest.fixture(scope="module", params=[c[0] for c in mg.CASES])
def case(request, oracle_lib, make_case):
    name, n_tok, samples, steps, tiny, run_steps = next(c for c in mg.CASES if c[0] == request.param)
    x, meta = make_case(n_tok, samples, steps, tiny)
    gold = load(name)
    assert int(gold["digest"][0]) == mg.input_digest(x), "synthetic inputs differ from the ones the fixture was made with"
    oracle_lib.setup(x, meta)
    return name, meta, gold, run_steps


def test_denoiser_checkpoints(case, oracle_lib):
    name, meta, gold, _ = case
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.clear_snapshots()
    for tag, (stop, bufs) in mg.STOPS.items():
        if stop:
            for b in bufs:
                oracle_lib.snapshot(stop, b)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    worst = {}
    for tag, (stop, bufs) in mg.STOPS.items():
        for b in bufs:
            got = oracle_lib.read("%s@%d" % (b, stop) if stop else b)
            err = driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)])
            worst["%s.%s" % (tag, b)] = err
    oracle_lib.clear_snapshots()
    assert worst["atom_init.QA"] <= EXACT_TOL and worst["atom_init.NTV"] <= EXACT_TOL, worst
    bad = {k: v for k, v in worst.items() if v > BF16_TOL}
    assert not bad, bad
    # the gate of the north star: one denoiser evaluation within 2e-2
    assert worst["final.OUT"] < 2e-2


def test_first_step_noise_and_augmentation(case, oracle_lib):
    """Positions after init (INIT stream), centring, rigid augmentation (AUGMENT) and churn (CHURN)."""
    name, meta, gold, run_steps = case
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=3, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("POS")), gold["step1.POS"]) <= EXACT_TOL
    assert driver.max_rel_err(picked(oracle_lib.read("XN")), gold["step1.XN"]) <= EXACT_TOL


def test_short_trajectory(case, oracle_lib):
    name, meta, gold, run_steps = case
    if name == "tiny" and os.environ.get("CCK_FAST_TESTS"):
        pytest.skip("20 oracle steps")
    oracle_lib.run(mode=0, nsteps=run_steps, seed=7)
    pos = oracle_lib.read("POS")
    assert np.isfinite(pos).all()
    assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < 2e-2


def test_heun_variant_against_reference_kernel(oracle_lib, make_case):
    """The Heun sampler (flag 128): the first half step (x1 in XN, the slope in GRAD), the first full
    step and a short trajectory against the reference kernel's."""
    name, n_tok, samples, steps, tiny, run_steps, churn = mg.HEUN_CASES[0]
    x, meta = make_case(n_tok, samples, steps, tiny, flags=synth.F_HEUN, churn=churn)
    gold = load(name)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    oracle_lib.setup(x, meta)
    half = mg.HEAD_PHASES + mg.DENOISE_PHASES + 1
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("XN")), gold["heun1.XN"]) < 2e-2
    assert driver.max_rel_err(picked(oracle_lib.read("GRAD")), gold["heun1.GRAD"]) < 2e-2
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half + mg.DENOISE_PHASES + 1, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("POS")), gold["step1.POS"]) < 2e-2
    if not os.environ.get("CCK_FAST_TESTS"):
        oracle_lib.run(mode=0, nsteps=run_steps, seed=7)
        pos = oracle_lib.read("POS")
        assert np.isfinite(pos).all()
        assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < 2e-2


def test_realign_variant_against_reference_kernel(oracle_lib, make_case):
    """REALIGN (flag 512): the denoised positions and the alignment's moments, the aligned Euler step
    and a short trajectory against the reference kernel's."""
    name, n_tok, samples, steps, tiny, run_steps = mg.REALIGN_CASES[0]
    x, meta = make_case(n_tok, samples, steps, tiny, flags=synth.F_REALIGN)
    gold = load(name)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    oracle_lib.setup(x, meta)
    half = mg.HEAD_PHASES + mg.DENOISE_PHASES + 1
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("GRAD")), gold["moments.GRAD"]) < 2e-2
    assert driver.max_rel_err(picked(oracle_lib.read("KAB")), gold["moments.KAB"]) < 2e-2
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half + 1, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("POS")), gold["step1.POS"]) < 2e-2
    if not os.environ.get("CCK_FAST_TESTS"):
        oracle_lib.run(mode=0, nsteps=run_steps, seed=7)
        assert driver.max_rel_err(picked(oracle_lib.read("POS")), gold["sample.POS"]) < 2e-2


@pytest.mark.parametrize("variant", [c[0] for c in mg.VARIANT_CASES])
def test_denoiser_variants_against_reference_kernel(variant, oracle_lib, make_case):
    """SCFINAL and IDSCALE: checkpoints of one denoiser call against the reference kernel's."""
    flags = dict(mg.VARIANT_CASES)[variant]
    x, meta = make_case(32, 1, 20, True, flags=flags)
    gold = load(variant)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    oracle_lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.clear_snapshots()
    for tag, (stop, bufs) in mg.variant_stops(variant).items():
        if stop:
            for b in bufs:
                oracle_lib.snapshot(stop, b)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    worst = {}
    for tag, (stop, bufs) in mg.variant_stops(variant).items():
        for b in bufs:
            got = oracle_lib.read("%s@%d" % (b, stop) if stop else b)
            worst["%s.%s" % (tag, b)] = driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)])
    oracle_lib.clear_snapshots()
    bad = {k: v for k, v in worst.items() if v > BF16_TOL}
    assert not bad, bad
    assert worst["final.OUT"] < 2e-2


def test_precise_mode_is_close_to_faithful_mode(case, oracle_lib):
    name, meta, gold, _ = case
    if name != "tiny":
        pytest.skip("one case is enough")
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE, precise=True)
    f32 = oracle_lib.read("OUT").copy()
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE, precise=False)
    assert driver.max_rel_err(oracle_lib.read("OUT"), f32) < 2e-2


def test_philox_known_properties(oracle_lib):
    """Counter-based: same counter and key give the same words; each field of the counter and each
    half of the key matters; normals come from the 24 high bits by Box-Muller."""
    w0, z0 = oracle_lib.philox(5, 3, 1, 0, 0x0123456789ABCDEF)
    w1, z1 = oracle_lib.philox(5, 3, 1, 0, 0x0123456789ABCDEF)
    assert (w0 == w1).all() and (z0 == z1).all()
    for other in [(6, 3, 1, 0), (5, 4, 1, 0), (5, 3, 2, 0), (5, 3, 1, 1)]:
        w, _ = oracle_lib.philox(*other, 0x0123456789ABCDEF)
        assert (w != w0).any()
    assert (oracle_lib.philox(5, 3, 1, 0, 0x0123456789ABCDEE)[0] != w0).any()
    assert (oracle_lib.philox(5, 3, 1, 0, 0x1123456789ABCDEF)[0] != w0).any()
    u1 = (np.float32((int(w0[0]) >> 8) + 1) * np.float32(2.0 ** -24)).astype(np.float32)
    u2 = np.float32(int(w0[1]) >> 8) * np.float32(2.0 ** -24)
    r = np.sqrt(np.float32(-2.0) * np.log(u1))
    assert np.isclose(z0[0], r * np.cos(np.float32(2 * np.pi) * u2), rtol=1e-5, atol=1e-6)
    # moments of many normals
    zs = np.array([oracle_lib.philox(i, 0, 0, 2, 42)[1] for i in range(4096)]).ravel()
    assert abs(zs.mean()) < 0.05 and abs(zs.std() - 1.0) < 0.05


def curand_words(counters, seed):
    """Raw Philox4x32-10 words of NVIDIA's own implementation (the cuRAND header built for the host,
    oracle/philox_curand.cpp): an implementation independent of both the sampler and the oracle."""
    import ctypes

    path = os.path.join(os.path.dirname(GOLDEN), "..", "oracle", "libphilox_curand.so")
    if not os.path.isfile(path):
        import subprocess

        subprocess.run(["make", "-C", os.path.dirname(path), os.path.abspath(path)], check=True)
    lib = ctypes.CDLL(os.path.abspath(path))
    lib.kat_curand_philox.argtypes = [ctypes.c_void_p] * 3
    lib.kat_curand_philox.restype = None
    key = np.array([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32)
    out = np.empty((len(counters), 4), dtype=np.uint32)
    for i, c in enumerate(counters):
        cc = np.array(c, dtype=np.uint32)
        lib.kat_curand_philox(cc.ctypes.data, key.ctypes.data, out[i].ctypes.data)
    return out


def philox_counters(n=1000, seed=2024):
    """Counters as the sampler forms them, (slot index, step, sample, stream), plus extreme words."""
    rng = np.random.default_rng(seed)
    c = np.stack([rng.integers(0, 50000, n), rng.integers(0, 201, n), rng.integers(0, 8, n), rng.integers(0, 3, n)], axis=1)
    edge = [[0, 0, 0, 0], [0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF], [1, 0, 0, 0], [0, 0, 0, 0x80000000]]
    return np.concatenate([c, np.array(edge)], axis=0).astype(np.uint64)


@pytest.mark.parametrize("seed", [0, 7, 0x0123456789ABCDEF, 0xFFFFFFFFFFFFFFFF])
def test_philox_words_are_curands(oracle_lib, seed):
    """Raw words, bit for bit: the oracle's Philox against cuRAND's on a thousand counters
    (reference: src/diffusion/rng.cuh:14-35; integer work is held to equality)."""
    counters = philox_counters()
    want = curand_words(counters, seed)
    got = np.array([oracle_lib.philox(int(c[0]), int(c[1]), int(c[2]), int(c[3]), seed)[0] for c in counters])
    assert np.array_equal(got, want)


def masked_case(make=synth.masked_bucket_case, _cache={}):
    if "x" not in _cache:
        _cache["x"] = make()
    return _cache["x"]


def test_masked_bucket_against_reference_kernel(oracle_lib):
    """A fold told by masks alone inside a larger bucket (the operator's ext[2] = 0 path): zero
    TMASK / QMASK / KMASK / ATOM_MASK / TAM in the padding and on masked real tokens, a partly filled
    last subset, the extra pair logits PLX present. Checkpoints, first-step noise and a short
    trajectory of the oracle against the reference kernel's."""
    x, meta = masked_case()
    gold = load("masked")
    assert int(gold["digest"][0]) == mg.input_digest(x)
    oracle_lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.clear_snapshots()
    for tag, (stop, bufs) in mg.MASKED_STOPS.items():
        if stop:
            for b in bufs:
                oracle_lib.snapshot(stop, b)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    worst = {}
    for tag, (stop, bufs) in mg.MASKED_STOPS.items():
        for b in bufs:
            got = oracle_lib.read("%s@%d" % (b, stop) if stop else b)
            worst["%s.%s" % (tag, b)] = driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)])
    oracle_lib.clear_snapshots()
    assert worst["atom_init.QA"] <= EXACT_TOL, worst
    assert not {k: v for k, v in worst.items() if v > BF16_TOL}, worst
    oracle_lib.run(mode=0, nsteps=int(gold["sample.steps"][0]), dbg_stop=3, seed=7)
    assert driver.max_rel_err(picked(oracle_lib.read("XN")), gold["step1.XN"]) <= EXACT_TOL
    if not os.environ.get("CCK_FAST_TESTS"):
        oracle_lib.run(mode=0, nsteps=int(gold["sample.steps"][0]), seed=7)
        assert driver.max_rel_err(picked(oracle_lib.read("POS")), gold["sample.POS"]) < 2e-2

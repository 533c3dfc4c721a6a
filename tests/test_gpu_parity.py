"""Parity of the CUDA path, called through the library's C ABI, against the CPU oracle on the same
seeded inputs and against the golden fixtures of the reference kernel. Floating point: the gate is
max |a-b| / max |b| <= 2e-2 for one denoiser evaluation in bf16 (the tolerance the benchmark
definition states); intermediate bf16 buffers are held to 1e-2, f32-only paths to 2e-6."""
import ctypes
import os
import sys

import numpy as np
import pytest

from mkharness import driver, synth

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden as mg  # noqa: E402
from test_oracle import load, picked  # noqa: E402

pytestmark = pytest.mark.gpu
BF16_TOL, EXACT_TOL, GATE = 1e-2, 2e-6, 2e-2
RMS_TOL = 5e-3  # RMS(a - b) / RMS(b) of a bf16 buffer: beside the global maximum, which large entries dominate


@pytest.fixture(scope="module")
def lib(product_lib_path):
    return driver.MkLib(product_lib_path)  # raises when the CUDA library is missing: no fallback


@pytest.mark.parametrize("shape", [(128, 256, 64, 256), (128, 128, 128, 128), (300, 384, 128, 128), (32, 64, 64, 64),
                                   (1000, 512, 256, 256), (2560, 3072, 768, 0), (2560, 768, 1536, 0), (77, 192, 320, 64)])
def test_gemm_door(lib, oracle_lib, shape):
    """The tcgen05 GEMM engine alone: f32 accumulation, so it agrees with the CPU to f32 rounding."""
    M, N, K, tile = shape
    rng = np.random.default_rng(M + N + K)
    a = synth.to_bf16(rng.standard_normal((M, K), dtype=np.float32))
    w = synth.to_bf16(rng.standard_normal((N, K), dtype=np.float32) / np.sqrt(K))
    assert driver.max_rel_err(lib.gemm_test(a, w, tile), oracle_lib.gemm(a, w)) < 1e-5


def test_gemm_linearity(lib):
    """At the benchmark's GEMM size: A·Wᵀ with W = [W1; W2] equals the two halves side by side, and a
    zero A gives exact zeros."""
    rng = np.random.default_rng(3)
    a = synth.to_bf16(rng.standard_normal((2560, 768), dtype=np.float32))
    w = synth.to_bf16(rng.standard_normal((512, 768), dtype=np.float32))
    c = lib.gemm_test(a, w, 256)
    assert (lib.gemm_test(a, w[:256], 256) == c[:, :256]).all() and (lib.gemm_test(a, w[256:], 128) == c[:, 256:]).all()
    assert (lib.gemm_test(np.zeros_like(a), w, 0) == 0).all()


@pytest.fixture(scope="module", params=[c[0] for c in mg.CASES])
def case(request, lib, oracle_lib, make_case):
    name, n_tok, samples, steps, tiny, run_steps = next(c for c in mg.CASES if c[0] == request.param)
    x, meta = make_case(n_tok, samples, steps, tiny)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    return name, meta, load(name), run_steps


def test_denoiser_checkpoints(case, lib, oracle_lib):
    name, meta, gold, _ = case
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.clear_snapshots()
    for tag, (stop, bufs) in mg.STOPS.items():
        if stop:
            for b in bufs:
                oracle_lib.snapshot(stop, b)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    vs_oracle, vs_ref, rms_oracle, rms_ref = {}, {}, {}, {}
    for tag, (stop, bufs) in mg.STOPS.items():
        lib.run(mode=1, dbg_stop=stop, xn=xn, t=mg.T_ONCE)
        for b in bufs:
            got = lib.read(b)
            want = oracle_lib.read("%s@%d" % (b, stop) if stop else b)
            vs_oracle["%s.%s" % (tag, b)] = driver.max_rel_err(got, want)
            rms_oracle["%s.%s" % (tag, b)] = driver.rms_rel_err(got, want)
            vs_ref["%s.%s" % (tag, b)] = driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)])
            rms_ref["%s.%s" % (tag, b)] = driver.rms_rel_err(picked(got), gold["%s.%s" % (tag, b)])
    oracle_lib.clear_snapshots()
    assert vs_oracle["atom_init.QA"] <= EXACT_TOL and vs_oracle["atom_init.NTV"] <= EXACT_TOL
    assert not {k: v for k, v in vs_oracle.items() if v > BF16_TOL}, vs_oracle
    assert not {k: v for k, v in vs_ref.items() if v > BF16_TOL}, vs_ref
    assert not {k: v for k, v in rms_oracle.items() if v > RMS_TOL}, rms_oracle
    assert not {k: v for k, v in rms_ref.items() if v > RMS_TOL}, rms_ref
    assert vs_oracle["final.OUT"] < GATE and vs_ref["final.OUT"] < GATE


def test_first_step_noise_matches_reference_and_oracle(case, lib, oracle_lib):
    name, meta, gold, run_steps = case
    lib.run(mode=0, nsteps=run_steps, dbg_stop=3, seed=7)
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=3, seed=7)
    for b in ("POS", "XN"):
        got = lib.read(b)
        assert driver.max_rel_err(got, oracle_lib.read(b)) <= EXACT_TOL
        assert driver.max_rel_err(picked(got), gold["step1." + b]) <= EXACT_TOL


def test_trajectory_and_determinism(case, lib, oracle_lib):
    name, meta, gold, run_steps = case
    lib.run(mode=0, nsteps=run_steps, seed=7)
    pos = lib.read("POS").copy()
    assert np.isfinite(pos).all()
    lib.run(mode=0, nsteps=run_steps, seed=7)
    assert (lib.read("POS") == pos).all(), "a fold must be bit-reproducible run to run"
    lib.run(mode=0, nsteps=run_steps, seed=8)
    assert (lib.read("POS") != pos).any(), "the seed keys the noise"
    assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < GATE
    oracle_lib.run(mode=0, nsteps=run_steps, seed=7)
    ref = oracle_lib.read("POS")
    assert driver.max_rel_err(pos, ref) < GATE
    rmsd = float(np.sqrt(((pos - ref).reshape(-1, 3) ** 2).sum(-1).mean()))
    print("%s: RMSD after %d steps vs oracle %.4f A" % (name, run_steps, rmsd))


def test_status_words_after_a_clean_run(case, lib):
    name, meta, gold, _ = case
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    st, where, bars = ctypes.c_uint(9), ctypes.c_uint(9), ctypes.c_uint(0)
    lib.lib.cck_last_status(ctypes.byref(st), ctypes.byref(where), ctypes.byref(bars))
    assert st.value == 0 and bars.value > 60  # one denoiser call: 2 barriers per token block on completion counters (7 without), ~25 around them


def test_operator_entry_point_matches_debug_api(lib, make_case):
    """cck_mk_sample (what the XLA FFI handler wraps) with caller-owned device buffers: same positions
    as the debug API's sampling run, zero rows past the real tokens, ext read on the device."""
    import torch

    x, meta = make_case(32, 1, 20, True)
    steps = 4
    lib.setup(x, meta)
    lib.run(mode=0, nsteps=steps, seed=11)
    want = lib.read("POS").copy()
    dev = [torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda() for a in x]
    ptrs = (ctypes.c_void_p * 74)(*[t.data_ptr() for t in dev])
    sizes = (ctypes.c_size_t * 74)(*[a.nbytes for a in x])
    ws_bytes = lib.workspace_bytes(x, meta, steps)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda").fill_(0xAB)  # handed over dirty
    out = torch.full((1, meta["N"], 24, 3), 7.0, dtype=torch.float32, device="cuda")
    ext = torch.tensor([meta["N"], meta["NS"], 1, 11, 0], dtype=torch.int32, device="cuda")
    f = lib.lib.cck_mk_sample
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                  ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.lib.cck_last_error.restype = ctypes.c_char_p
    stream = torch.cuda.current_stream().cuda_stream
    rc = f(stream, ext.data_ptr(), ptrs, sizes, 74, out.data_ptr(), meta["N"], ws.data_ptr(), ws_bytes, 1, steps, 0)
    assert rc == 0, lib.lib.cck_last_error()
    torch.cuda.synchronize()
    assert (out.cpu().numpy().ravel() == want).all()


@pytest.mark.parametrize("variant", [c[0] for c in mg.VARIANT_CASES])
def test_denoiser_variants(variant, lib, oracle_lib, make_case):
    """SCFINAL and IDSCALE: one denoiser call against the oracle (every buffer of the checkpoints)
    and against the reference kernel's fixture; the plain denoiser must differ."""
    flags = dict(mg.VARIANT_CASES)[variant]
    x, meta = make_case(32, 1, 20, True, flags=flags)
    gold = load(variant)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    for tag, (stop, bufs) in mg.variant_stops(variant).items():
        lib.run(mode=1, dbg_stop=stop, xn=xn, t=mg.T_ONCE)
        oracle_lib.run(mode=1, dbg_stop=stop, xn=xn, t=mg.T_ONCE)
        for b in bufs:
            got = lib.read(b)
            assert driver.max_rel_err(got, oracle_lib.read(b)) < GATE, (tag, b)
            assert driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)]) < GATE, (tag, b)
    out = lib.read("OUT").copy()
    if flags == synth.F_ATOB:
        return  # its inputs have other shapes: there is no "same inputs without the bit"
    xm = [a.copy() for a in x]  # the same inputs without the bit
    xm[synth.IN["MISC"]][4] = 0.0
    lib.setup(xm, meta)
    lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    assert driver.max_rel_err(lib.read("OUT"), out) > 1e-3


def test_variant_flags_combine(lib, oracle_lib, make_case):
    """All built variant bits at once, two sampling steps: the CUDA path against the oracle."""
    flags = synth.F_HEUN | synth.F_SCFINAL | synth.F_IDSCALE | synth.F_QKNORM | synth.F_CHAIN_K | synth.F_PARALLEL | synth.F_ATOB | synth.F_CHIRAL
    x, meta = make_case(32, 1, 8, True, flags=flags, churn=0.5)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    lib.run(mode=0, nsteps=2, seed=3)
    oracle_lib.run(mode=0, nsteps=2, seed=3)
    pos = lib.read("POS")
    assert np.isfinite(pos).all()
    assert driver.max_rel_err(pos, oracle_lib.read("POS")) < GATE


def test_realign_variant(lib, oracle_lib, make_case):
    """Flag 512: the denoised positions and the alignment's moments, the aligned Euler step and a
    short trajectory against the oracle and the reference kernel's fixture."""
    name, n_tok, samples, steps, tiny, run_steps = mg.REALIGN_CASES[0]
    x, meta = make_case(n_tok, samples, steps, tiny, flags=synth.F_REALIGN)
    gold = load(name)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    half = mg.HEAD_PHASES + mg.DENOISE_PHASES + 1
    lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    for b in ("GRAD", "KAB"):
        got = lib.read(b)
        assert driver.max_rel_err(got, oracle_lib.read(b)) < GATE, b
        assert driver.max_rel_err(picked(got), gold["moments." + b]) < GATE, b
    lib.run(mode=0, nsteps=run_steps, dbg_stop=half + 1, seed=7)
    assert driver.max_rel_err(picked(lib.read("POS")), gold["step1.POS"]) < GATE
    lib.run(mode=0, nsteps=run_steps, seed=7)
    pos = lib.read("POS").copy()
    assert np.isfinite(pos).all()
    assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < GATE


def test_heun_variant(lib, oracle_lib, make_case):
    """Flag 128: two denoiser calls per step. The half step, the full step and a short trajectory
    against the oracle and the reference kernel's fixture; the plain sampler must differ."""
    name, n_tok, samples, steps, tiny, run_steps, churn = mg.HEUN_CASES[0]
    x, meta = make_case(n_tok, samples, steps, tiny, flags=synth.F_HEUN, churn=churn)
    gold = load(name)
    assert int(gold["digest"][0]) == mg.input_digest(x)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    half = mg.HEAD_PHASES + mg.DENOISE_PHASES + 1
    lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    oracle_lib.run(mode=0, nsteps=run_steps, dbg_stop=half, seed=7)
    for b in ("XN", "GRAD"):
        got = lib.read(b)
        assert driver.max_rel_err(got, oracle_lib.read(b)) < GATE, b
        assert driver.max_rel_err(picked(got), gold["heun1." + b]) < GATE, b
    lib.run(mode=0, nsteps=run_steps, dbg_stop=half + mg.DENOISE_PHASES + 1, seed=7)
    assert driver.max_rel_err(picked(lib.read("POS")), gold["step1.POS"]) < GATE
    lib.run(mode=0, nsteps=run_steps, seed=7)
    pos = lib.read("POS").copy()
    assert np.isfinite(pos).all()
    assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < GATE
    def barriers():
        st, where, bars = ctypes.c_uint(9), ctypes.c_uint(9), ctypes.c_uint(0)
        lib.lib.cck_last_status(ctypes.byref(st), ctypes.byref(where), ctypes.byref(bars))
        assert st.value == 0
        return bars.value

    heun_barriers = barriers()
    x0, meta0 = make_case(n_tok, samples, steps, tiny)
    lib.setup(x0, meta0)
    lib.run(mode=0, nsteps=run_steps, seed=7)
    assert driver.max_rel_err(lib.read("POS"), pos) > 1e-3, "the Euler path gives another trajectory"
    assert heun_barriers > 1.9 * barriers(), "two denoiser calls per step"


def test_real_extents_inside_a_larger_bucket(lib, make_case):
    """The operator compiles per shape bucket and passes the real extents in ext (device memory).
    A 48-token, 12-subset fold laid out in a 64-token, 16-subset bucket must give the positions of
    the exact-shape run, whatever sits in the padding (zeros, or NaN where nothing may be read),
    through the debug API and through cck_mk_sample (which also zeroes the rows past the real tokens)."""
    import torch

    x, meta = make_case(48, 2, 8, False)
    S, N, steps, seed = meta["S"], meta["N"], 3, 5
    lib.setup(x, meta)
    lib.run(mode=0, nsteps=steps, seed=seed)
    exact = lib.read("POS").copy()
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    exact_out = lib.read("OUT").copy()
    for poison in (False, True):
        xb, mb = synth.pad_to_bucket(x, meta, 64, 16, poison=poison)
        lib.setup(xb, mb)
        lib.set_extent(N, meta["NS"])
        lib.run(mode=0, nsteps=steps, seed=seed)
        got = lib.read("POS")[: exact.size]
        assert np.isfinite(got).all()
        assert driver.max_rel_err(got, exact) <= 1e-6, "poison=%s" % poison
        xnb = np.zeros(S * mb["N"] * 24 * 3, dtype=np.float32)
        xnb[: xn.size] = xn.ravel()
        lib.run(mode=1, xn=xnb, t=mg.T_ONCE)
        assert driver.max_rel_err(lib.read("OUT")[: exact_out.size], exact_out) <= 1e-6
    # the operator entry point with ext = {48, 12, exact, seed, 0} on the bucket's buffers
    dev = [torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda() for a in xb]
    ptrs = (ctypes.c_void_p * 74)(*[t.data_ptr() for t in dev])
    sizes = (ctypes.c_size_t * 74)(*[a.nbytes for a in xb])
    ws_bytes = lib.workspace_bytes(xb, mb, steps)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda").fill_(0xFF)  # NaN patterns everywhere
    out = torch.full((S, mb["N"], 24, 3), 7.0, dtype=torch.float32, device="cuda")
    ext = torch.tensor([N, meta["NS"], 1, seed, 0], dtype=torch.int32, device="cuda")
    f = lib.lib.cck_mk_sample
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                  ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    rc = f(torch.cuda.current_stream().cuda_stream, ext.data_ptr(), ptrs, sizes, 74, out.data_ptr(), mb["N"], ws.data_ptr(),
           ws_bytes, S, steps, 0)
    assert rc == 0
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert driver.max_rel_err(o[:, :N].ravel(), exact) <= 1e-6
    assert (o[:, N:] == 0).all()
    lib.lib.mk_set_extent(0, 0)


@pytest.mark.parametrize("n_tok,samples", [(160, 3), (256, 2)])
def test_completion_counters_match_barriers(lib, make_case, n_tok, samples):
    """Inside a token block QKVG -> attention -> WO and W1 -> W2 run without grid barriers, a unit
    waiting for the completion counters of the rows it reads (mk_set_flow, on by default). The same
    units compute the same values in another order: positions are bit-identical to the run on
    barriers. 160 tokens: samples do not start on a 128-row block, so blocks of rows and blocks of
    queries straddle; 3 steps reuse every counter 72 times per sample set."""
    x, meta = make_case(n_tok, samples, 8, False)
    lib.setup(x, meta)
    got = {}
    try:
        for on in (True, False):
            lib.set_flow(on)
            lib.run(mode=0, nsteps=3, seed=11)
            got[on] = lib.read("POS").copy()
            xn = synth.noisy_positions(meta, mg.T_ONCE)
            lib.run(mode=1, xn=xn, t=mg.T_ONCE)
            got[on, "once"] = lib.read("OUT").copy()
    finally:
        lib.set_flow(True)
    assert np.isfinite(got[True]).all()
    assert np.array_equal(got[True], got[False])
    assert np.array_equal(got[True, "once"], got[False, "once"])


@pytest.mark.parametrize("n_tok,samples", [(256, 5), (512, 5), (1024, 1), (1024, 5)])
def test_full_size_denoiser_against_oracle(lib, oracle_lib, make_case, n_tok, samples):
    """The benchmark's own shapes (256 and 512 tokens x 5 samples, 1024 tokens x 1 and x 5): one denoiser
    evaluation on the GPU against the CPU oracle on the same seeded inputs, within the stated 2e-2,
    plus what needs no oracle at this size: a short trajectory is finite, bit-reproducible run to run,
    and the same on completion counters as on grid barriers."""
    x, meta = make_case(n_tok, samples, 8, False)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    got = lib.read("OUT").copy()
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    err = driver.max_rel_err(got, oracle_lib.read("OUT"))
    print("N=%d S=%d: one denoiser evaluation, max rel err vs oracle %.2e" % (n_tok, samples, err))
    assert err < GATE
    pos = {}
    try:
        for on in (True, True, False):
            lib.set_flow(on)
            lib.run(mode=0, nsteps=2, seed=5)
            p = lib.read("POS").copy()
            assert np.isfinite(p).all()
            if on in pos:
                assert np.array_equal(pos[on], p), "a fold must be bit-reproducible run to run"
            pos[on] = p
    finally:
        lib.set_flow(True)
    assert np.array_equal(pos[True], pos[False])


def test_stress_size_properties(lib, make_case):
    """2048 tokens, one sample (the largest configuration): 16 blocks of queries per head, a pair-logit
    table of 3.2 GB. No oracle at this size; the trajectory is finite, bit-reproducible, the same on
    completion counters as on barriers, and another seed gives another trajectory."""
    x, meta = make_case(2048, 1, 8, False)
    lib.setup(x, meta)
    pos = {}
    try:
        for on, seed in ((True, 3), (True, 3), (False, 3), (True, 4)):
            lib.set_flow(on)
            lib.run(mode=0, nsteps=2, seed=seed)
            p = lib.read("POS").copy()
            assert np.isfinite(p).all()
            if (on, seed) in pos:
                assert np.array_equal(pos[on, seed], p)
            pos[on, seed] = p
    finally:
        lib.set_flow(True)
    assert np.array_equal(pos[True, 3], pos[False, 3])
    assert not np.array_equal(pos[True, 3], pos[True, 4])


def test_headline_size_against_reference_kernel(lib, make_case):
    """512 tokens x 5 samples: one denoiser evaluation of this library against the reference's own
    CUDA kernel (its diffusion.cu compiled unmodified for sm_100 under oracle/_ref) on the same inputs."""
    if not os.path.isfile(driver.REFERENCE_LIB):
        pytest.skip("oracle/_ref/libref_sm100.so is not built on this machine")
    x, meta = make_case(512, 5, 8, False)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    lib.setup(x, meta)
    lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    got = lib.read("OUT").copy()
    lib.teardown()
    ref = driver.MkLib(driver.REFERENCE_LIB)
    ref.setup(x, meta)
    ref.run(mode=1, xn=xn, t=mg.T_ONCE)
    want = ref.read("OUT").copy()
    ref.teardown()
    err, rms = driver.max_rel_err(got, want), driver.rms_rel_err(got, want)
    print("512 x 5 vs the reference kernel: max rel err %.2e, rms rel err %.2e" % (err, rms))
    assert err < GATE and rms < RMS_TOL


def test_philox_words_bit_exact(lib, oracle_lib):
    """Raw Philox4x32-10 words on the device, bit for bit against cuRAND's implementation and the
    oracle's; the Box-Muller normals to f32 resolution (device logf/cosf against libm)."""
    from test_oracle import curand_words, philox_counters

    f = lib.lib.mk_philox_test
    f.argtypes = [ctypes.c_uint32] * 4 + [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    seed = 0x0123456789ABCDEF
    counters = philox_counters(300)
    want = curand_words(counters, seed)
    w, z = np.empty(4, dtype=np.uint32), np.empty(4, dtype=np.float32)
    for c, ww in zip(counters, want):
        assert f(int(c[0]), int(c[1]), int(c[2]), int(c[3]), seed, w.ctypes.data, z.ctypes.data) == 0
        assert np.array_equal(w, ww), c
        ow, oz = oracle_lib.philox(int(c[0]), int(c[1]), int(c[2]), int(c[3]), seed)
        assert np.array_equal(w, ow)
        assert np.allclose(z, oz, rtol=2e-6, atol=2e-6)


def test_token_gather_is_exact(lib, make_case):
    """decoder_init, qa = (skip + tb[token of the atom])·QMASK, is an f32 gather and add: the CUDA
    path's QA equals what numpy forms from its own SKIP and TB buffers, element for element."""
    x, meta = make_case(48, 2, 8, False)
    lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    stop = 12 + 7 * 24 + 3  # pair build, atom init, 9 encoder phases, aggregation, the token blocks, final LN, broadcast, decoder init
    lib.run(mode=1, dbg_stop=stop, xn=xn, t=mg.T_ONCE)
    S, N, A = meta["S"], meta["N"], meta["A"]
    qa = lib.read("QA").reshape(S, A, 128)
    skip = lib.read("SKIP").reshape(S, A, 128)
    tb = lib.read("TB").reshape(S, N, 128)
    tok2q, qmask = x[synth.IN["TOK2Q"]], x[synth.IN["QMASK"]]
    want = skip.copy()
    has = tok2q >= 0
    want[:, has] = skip[:, has] + tb[:, tok2q[has] // 24]
    want *= qmask[None, :, None]
    assert np.array_equal(qa, want)


def test_masked_bucket(lib, oracle_lib):
    """A fold told by masks alone inside a larger bucket (the operator's ext[2] = 0 path: the bucket's
    extents run and zero masks do the work), a partly filled last subset, masked real tokens and
    the extra pair logits PLX: the CUDA path against the oracle and the reference kernel's fixture."""
    from test_oracle import masked_case

    x, meta = masked_case()
    gold = load("masked")
    assert int(gold["digest"][0]) == mg.input_digest(x)
    lib.setup(x, meta)
    oracle_lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    oracle_lib.clear_snapshots()
    for tag, (stop, bufs) in mg.MASKED_STOPS.items():
        if stop:
            for b in bufs:
                oracle_lib.snapshot(stop, b)
    oracle_lib.run(mode=1, xn=xn, t=mg.T_ONCE)
    vs_oracle, vs_ref = {}, {}
    for tag, (stop, bufs) in mg.MASKED_STOPS.items():
        lib.run(mode=1, dbg_stop=stop, xn=xn, t=mg.T_ONCE)
        for b in bufs:
            got = lib.read(b)
            vs_oracle["%s.%s" % (tag, b)] = driver.max_rel_err(got, oracle_lib.read("%s@%d" % (b, stop) if stop else b))
            vs_ref["%s.%s" % (tag, b)] = driver.max_rel_err(picked(got), gold["%s.%s" % (tag, b)])
    oracle_lib.clear_snapshots()
    assert vs_oracle["atom_init.QA"] <= EXACT_TOL
    assert not {k: v for k, v in vs_oracle.items() if v > BF16_TOL}, vs_oracle
    assert not {k: v for k, v in vs_ref.items() if v > BF16_TOL}, vs_ref
    steps = int(gold["sample.steps"][0])
    lib.run(mode=0, nsteps=steps, dbg_stop=3, seed=7)
    assert driver.max_rel_err(picked(lib.read("XN")), gold["step1.XN"]) <= EXACT_TOL
    lib.run(mode=0, nsteps=steps, seed=7)
    pos = lib.read("POS").copy()
    assert np.isfinite(pos).all()
    assert driver.max_rel_err(picked(pos), gold["sample.POS"]) < GATE
    # the same fold with the pair logits PLX absent gives other positions: the input is read
    xm = [a.copy() for a in x]
    xm[synth.IN["PLX"]] = np.zeros(2, dtype=np.uint16)
    lib.setup(xm, meta)
    lib.run(mode=0, nsteps=steps, seed=7)
    assert driver.max_rel_err(lib.read("POS"), pos) > 1e-4


def test_pipelines_of_the_token_attention_do_not_depend_on_their_skew(lib, make_case):
    """The token attention keeps two items in flight per CTA as independent pipelines; whatever their
    relative timing, a fold's result is the same bit for bit. The test hook delays the second pipeline
    by a few microseconds (part of an item), on grid barriers and on completion counters, at a size
    where every CTA has both pipelines busy."""
    x, meta = make_case(512, 5, 8, False)
    lib.setup(x, meta)
    xn = synth.noisy_positions(meta, mg.T_ONCE)
    skew = lib.lib.mk_set_attn_skew
    want = None
    try:
        for flow in (False, True):
            lib.set_flow(flow)
            for cycles in (0, 3000, 10000):
                skew(cycles)
                lib.run(mode=1, xn=xn, t=mg.T_ONCE)
                out = lib.read("OUT").copy()
                if want is None:
                    want = out
                assert np.array_equal(out, want), (flow, cycles)
    finally:
        skew(0)
        lib.set_flow(True)


def test_waits_give_up_and_the_launch_ends(lib, make_case):
    """Every wait in the kernel is bounded. With the limit shortened to about a millisecond: (1) a thread
    that waits on an mbarrier nothing arrives at gives up and the kernel ends with status 2; (2) a fold
    whose grid barriers expect one arrival too many gives up at its first barrier: every CTA leaves
    the schedule, the launch ends normally with status 1 and the operator's output is NaN throughout
    instead of looking like coordinates; (3) the next ordinary fold is correct (nothing was left behind:
    TMEM freed, no flag stuck)."""
    import torch

    ms = ctypes.c_float(0)
    f = lib.lib.mk_wait_test
    f.argtypes = [ctypes.c_longlong, ctypes.POINTER(ctypes.c_float)]
    assert f(1 << 21, ctypes.byref(ms)) == 2  # ST_PIPE_TIMEOUT
    assert ms.value < 100.0
    x, meta = make_case(32, 1, 20, True)
    lib.setup(x, meta)
    lib.run(mode=0, nsteps=2, seed=3)
    want = lib.read("POS").copy()
    wt = lib.lib.mk_set_wait_test
    wt.argtypes = [ctypes.c_longlong, ctypes.c_int]
    st, where, bars = ctypes.c_uint(9), ctypes.c_uint(9), ctypes.c_uint(9)
    try:
        wt(1 << 21, 1)
        with pytest.raises(RuntimeError):
            lib.run(mode=0, nsteps=2, seed=3)
        lib.lib.cck_last_status(ctypes.byref(st), ctypes.byref(where), ctypes.byref(bars))
        assert st.value == 1 and where.value == 0  # ST_BARRIER_TIMEOUT at the first barrier
        # the operator entry point: the status is in the workspace's control words, the output says so too
        dev = [torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda() for a in x]
        ptrs = (ctypes.c_void_p * 74)(*[t.data_ptr() for t in dev])
        sizes = (ctypes.c_size_t * 74)(*[a.nbytes for a in x])
        ws_bytes = lib.workspace_bytes(x, meta, 2)
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
        out = torch.full((1, meta["N"], 24, 3), 7.0, dtype=torch.float32, device="cuda")
        ext = torch.tensor([meta["N"], meta["NS"], 1, 3, 0], dtype=torch.int32, device="cuda")
        g = lib.lib.cck_mk_sample
        g.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                      ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        assert g(torch.cuda.current_stream().cuda_stream, ext.data_ptr(), ptrs, sizes, 74, out.data_ptr(), meta["N"],
                 ws.data_ptr(), ws_bytes, 1, 2, 0) == 0  # enqueued; the failure shows after synchronising
        torch.cuda.synchronize()
        words = ws[:16].view(torch.int32).cpu().numpy()
        assert words[1] == 1  # the control words: {barrier, status, where, -}
        assert torch.isnan(out).all()
    finally:
        wt(0, 0)
    lib.run(mode=0, nsteps=2, seed=3)
    assert np.array_equal(lib.read("POS"), want)

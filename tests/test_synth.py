"""The synthetic input generator: layouts the kernels and the oracle rely on."""
import numpy as np

from mkharness import synth


def test_order_matches_the_operator_signature():
    assert synth.IN_NAMES[0] == "SIGMA" and synth.IN_NAMES[73] == "MISC"
    assert synth.IN["WQKVG"] == 19 and synth.IN["ENC_AMODS"] == 38 and synth.IN["DEC_AMODS"] == 46
    assert synth.IN["PCS"] == 60 and synth.IN["PLX"] == 64


def test_bf16_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], dtype=np.float32)
    b = synth.to_bf16(x)
    assert b[0] == 0x3F80
    assert b[1] == 0x3F80  # tie, rounds to even
    assert b[2] == 0x3F82  # tie, rounds to even (up)
    assert np.allclose(synth.from_bf16(b)[3], -2.5)


def test_karras_schedule_ends():
    s = synth.karras_sigmas(200)
    assert len(s) == 201
    assert np.isclose(s[0], 16 * 160.0, rtol=1e-5) and np.isclose(s[-1], 16 * 4e-4, rtol=1e-4)
    assert (np.diff(s) < 0).all()


def test_atom_layout(make_case):
    x, meta = make_case(48, 2, 8, False)
    N, A = meta["N"], meta["A"]
    assert A == 8 * N and meta["NS"] * 32 == A
    tok2q, q2ta = x[synth.IN["TOK2Q"]], x[synth.IN["Q2TA"]]
    assert (q2ta[tok2q] == np.arange(A)).all()
    per_tok = np.bincount(tok2q // 24, minlength=N)
    assert per_tok.min() >= 5 and per_tok.max() <= 14
    q2k = x[synth.IN["Q2K"]]
    assert q2k.shape == (meta["NS"], 128) and q2k.max() < A
    assert (x[synth.IN["KMASK"]] == (q2k >= 0)).all()


def test_apl_swizzle_matches_the_oracle_index(oracle_lib):
    rng = np.random.default_rng(0)
    NS, nk = 3, 128
    apl = rng.standard_normal((3, NS, 4, 32, nk)).astype(np.float32)
    sw = synth.apl_swizzle(apl).ravel()
    for (b, u, h, q, j) in [(0, 0, 0, 0, 0), (1, 2, 3, 17, 99), (2, 1, 2, 31, 127), (0, 2, 1, 8, 8), (2, 0, 3, 15, 16)]:
        idx = oracle_lib.lib.orc_apl_index(NS, nk, b, u, h, q, j)
        assert sw[idx] == apl[b, u, h, q, j]

"""Seeded synthetic inputs for the diffusion sampler: the 74 input buffers in the operator's order.

The reference receives these buffers from an external preparation step that is not part of its
tree, so this module states the layouts from how the reference kernel indexes each pointer
(src/diffusion/dims.cuh:61-74 for the order; src/diffusion/host.cuh:74-89 for the widths that are
derived from byte sizes). Distributions follow the benchmark description: s_trunk, z ~ N(0,1),
reference coordinates as a 3.8 A random-walk chain plus N(0, 1.5 A) atom offsets, LeCun-normal
weights, Karras sigma schedule.
"""
import numpy as np

IN_NAMES = (
    "SIGMA SC_BASE FOURIER_W FOURIER_B NOISE_LN WN "
    "ST0_S ST0_O ST0_W1 ST0_W2 ST1_S ST1_O ST1_W1 ST1_W2 "
    "WM1 BM1 WM2 BM2 WSE "
    "WQKVG BQ WO W1 W2 PC TMASK WTB "
    "WPOS SCQ QMASK KMASK Q2K TOK2Q Q2TA ATOM_MASK TAM WAGGR WUPD "
    "ENC_AMODS ENC_APL ENC_WQG ENC_BQ ENC_WKV ENC_WO ENC_W1 ENC_W2 "
    "DEC_AMODS DEC_APL DEC_WQG DEC_BQ DEC_WKV DEC_WO DEC_W1 DEC_W2 "
    "NOISE_LNO SE_B TB_B UPD_B SCF ROPE "
    "PCS PLW PLB PLWS PLX "
    "TQKN EQKN DQKN CHIR_W CHIR_C CHIR_A CHIR_PTR CHIR_IDX "
    "MISC"
).split()
IN = {name: i for i, name in enumerate(IN_NAMES)}
assert len(IN_NAMES) == 74

TOK_C, HEADS, QKVG, TOK_HIDDEN = 768, 16, 3072, 1536
ATOM_C, ATOM_HEADS, SUBSET, NK, SLOTS = 128, 4, 32, 128, 24
SIGMA_DATA = 16.0


def to_bf16(x):
    """float32 -> raw bf16 bits, round to nearest even (src/diffusion/frag.cuh:52-56). Large arrays
    (finite values: the same bits either way) go through torch's conversion, which runs on all host
    threads; the benchmark's pair representation alone has 10^8 elements."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    if a.size >= 1 << 22:
        try:
            import torch

            return torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        except ImportError:
            pass
    u = a.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def karras_sigmas(steps, sigma_data=SIGMA_DATA, s_max=160.0, s_min=4e-4, rho=7.0):
    i = np.arange(steps + 1, dtype=np.float64) / steps
    s = sigma_data * (s_max ** (1 / rho) + i * (s_min ** (1 / rho) - s_max ** (1 / rho))) ** rho
    return s.astype(np.float32)


def atoms_per_token(n_token, rng, tiny):
    if tiny:
        return np.full(n_token, 8, dtype=np.int64)
    cnt = rng.integers(5, 15, size=n_token)
    total = 8 * n_token
    # rebalance inside [5, 14] until the total is exact
    while cnt.sum() != total:
        i = rng.integers(0, n_token)
        if cnt.sum() > total and cnt[i] > 5:
            cnt[i] -= 1
        elif cnt.sum() < total and cnt[i] < 14:
            cnt[i] += 1
    return cnt


def apl_swizzle(apl):
    """[..., 32 queries, nk keys] -> the per-16x16-tile [lane][value] order the atom attention reads
    (src/diffusion/frag.cuh:127-143, src/diffusion/attention.cuh:323-324, :389)."""
    *lead, nq, nk = apl.shape
    t = apl.reshape(*lead, nq // 16, 16, nk // 16, 16)  # qt, r, kt, c
    t = np.moveaxis(t, -3, -2)  # qt, kt, r, c
    r = np.arange(16)[:, None]
    c = np.arange(16)[None, :]
    lane = (r % 8) * 4 + (c % 8) // 2
    slot = (c // 8) * 4 + (r // 8) * 2 + (c & 1)
    out = np.empty(t.shape[:-2] + (256,), dtype=apl.dtype)
    out[..., (lane * 8 + slot).ravel()] = t.reshape(t.shape[:-2] + (256,))
    return np.ascontiguousarray(out)


F_REALIGN, F_HEUN, F_SCFINAL, F_IDSCALE, F_CHIRAL, F_PARALLEL, F_QKNORM, F_ATOB, F_CHAIN_K = 512, 128, 64, 32, 16, 8, 4, 2, 1  # the variant bits that are built (src/diffusion/dims.cuh:46-57)


def make_inputs(n_token, samples=1, steps=200, seed=0, tiny=False, nb=24, cs=384, plc=128,
                gamma_min=1.0, flags=0, churn=0.0):
    """Returns (list of 74 contiguous numpy arrays, meta dict). `flags` and `churn` travel in MISC
    (the debug API reads the variant bits from there; the operator gets them as an attribute)."""
    rng = np.random.default_rng(seed)
    N = n_token
    cnt = atoms_per_token(N, rng, tiny)
    A = int(cnt.sum())
    assert A % SUBSET == 0
    NS = A // SUBSET
    tok_of_atom = np.repeat(np.arange(N), cnt)
    idx_in_tok = np.concatenate([np.arange(c) for c in cnt])

    def normal(*shape, std=1.0):
        a = rng.standard_normal(shape, dtype=np.float32)
        a *= np.float32(std)
        return a

    def lecun_bf(*shape):
        return to_bf16(normal(*shape, std=1.0 / np.sqrt(shape[-1])))

    x = [None] * 74

    def put(name, arr):
        x[IN[name]] = np.ascontiguousarray(arr)

    # geometry and index maps
    tok2q = (tok_of_atom * SLOTS + idx_in_tok).astype(np.int32)
    q2ta = np.full(N * SLOTS, -1, dtype=np.int32)
    q2ta[tok2q] = np.arange(A, dtype=np.int32)
    q2k = (np.arange(NS)[:, None] * SUBSET - 48 + np.arange(NK)[None, :]).astype(np.int32)
    q2k[(q2k < 0) | (q2k >= A)] = -1
    put("TOK2Q", tok2q)
    put("Q2TA", q2ta)
    put("Q2K", q2k)
    put("QMASK", np.ones(A, dtype=np.float32))
    put("KMASK", (q2k >= 0).astype(np.float32))
    put("ATOM_MASK", (q2ta >= 0).astype(np.float32))
    put("TAM", (q2ta >= 0).astype(np.float32))
    put("TMASK", np.ones(N, dtype=np.float32))

    # reference coordinates: 3.8 A random-walk chain of tokens + N(0, 1.5 A) atom offsets
    step_dir = normal(N, 3)
    step_dir /= np.linalg.norm(step_dir, axis=1, keepdims=True)
    chain = np.cumsum(3.8 * step_dir, axis=0)
    ref = chain[tok_of_atom] + normal(A, 3, std=1.5)

    # schedule and scalars
    put("SIGMA", karras_sigmas(steps))
    put("MISC", np.array([0.8, gamma_min, 1.003, 1.5, float(flags), churn], dtype=np.float32))

    # single conditioning
    put("SC_BASE", normal(N, cs))
    put("FOURIER_W", normal(256))
    put("FOURIER_B", rng.random(256, dtype=np.float32))
    put("NOISE_LN", 1.0 + normal(256, std=0.1))
    put("NOISE_LNO", normal(256, std=0.1))
    put("WN", normal(256, cs, std=1.0 / 16.0))
    for i in range(2):
        put("ST%d_S" % i, 1.0 + normal(cs, std=0.1))
        put("ST%d_O" % i, normal(cs, std=0.1))
        put("ST%d_W1" % i, lecun_bf(4 * cs, cs))
        put("ST%d_W2" % i, lecun_bf(cs, 2 * cs))
    put("WM1", lecun_bf(nb * 4 * TOK_C, cs))
    put("BM1", normal(nb * 4 * TOK_C, std=0.1))
    put("WM2", lecun_bf(nb * 2 * TOK_C, cs))
    put("BM2", -2.0 + normal(nb * 2 * TOK_C, std=0.1))
    put("WSE", lecun_bf(TOK_C, cs))
    put("SE_B", normal(TOK_C, std=0.1))
    if flags & F_SCFINAL:  # drawn only for the variant, so that the plain inputs stay as they were
        put("SCF", np.concatenate([1.0 + normal(cs, std=0.2), normal(cs, std=0.2)]).astype(np.float32))
    else:
        put("SCF", np.concatenate([np.ones(cs), np.zeros(cs)]).astype(np.float32))

    # token transformer
    put("WQKVG", lecun_bf(nb, QKVG, TOK_C))
    put("BQ", normal(nb, TOK_C, std=0.1))
    put("WO", lecun_bf(nb, TOK_C, TOK_C))
    # ATOB: units of 96 rows [gate 32 | proj 32 | a_to_b 32] instead of 64
    put("W1", lecun_bf(nb, (3 if flags & F_ATOB else 2) * TOK_HIDDEN, TOK_C))
    put("W2", lecun_bf(nb, TOK_C, TOK_HIDDEN))
    put("WTB", lecun_bf(ATOM_C, TOK_C))
    put("TB_B", normal(ATOM_C, std=0.1))
    put("WAGGR", lecun_bf(TOK_C, ATOM_C))

    # pair representation and its folded LayerNorm projection
    z = to_bf16(normal(N, N, plc))
    zf = from_bf16(z).astype(np.float64)
    mean = zf.mean(-1)
    rstd = 1.0 / np.sqrt(zf.var(-1) + 1e-5)
    put("PC", z)
    put("PCS", np.stack([mean, rstd], -1).astype(np.float32))
    plw = lecun_bf(nb, HEADS, plc)
    put("PLW", plw)
    put("PLWS", from_bf16(plw).astype(np.float64).sum(-1).astype(np.float32).reshape(-1))
    put("PLB", normal(nb * HEADS, std=0.1))
    put("PLX", np.zeros(2, dtype=np.uint16))  # absent: any size other than N*N*2 bytes

    # atom path
    put("WPOS", normal(3, ATOM_C, std=1.0 / np.sqrt(3.0)))
    feat = np.concatenate([ref / 10.0, normal(A, 13)], axis=1).astype(np.float32)  # 16 per atom
    put("SCQ", feat @ normal(16, ATOM_C, std=0.25))
    put("WUPD", normal(3, ATOM_C, std=1.0 / np.sqrt(ATOM_C)))
    put("UPD_B", normal(3, std=0.1))

    def pair_logits():
        # [3][NS][4][32][NK], natural-log units: a distance kernel per head plus noise; -1e9 where
        # the window has no key
        out = np.empty((3, NS, ATOM_HEADS, SUBSET, NK), dtype=np.float32)
        wh = normal(3, ATOM_HEADS)
        for u in range(NS):
            qi = np.arange(u * SUBSET, (u + 1) * SUBSET)
            ki = q2k[u]
            kk = np.clip(ki, 0, A - 1)
            dist2 = ((ref[qi][:, None, :] - ref[kk][None, :, :]) ** 2).sum(-1)
            base = 1.0 / (1.0 + dist2 / 16.0)
            out[:, u] = wh[:, :, None, None] * base[None, None] + normal(3, ATOM_HEADS, SUBSET, NK, std=0.5)
            out[:, u][..., ki < 0] = -1e9
        return apl_swizzle(out)

    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    for side in ("ENC", "DEC"):
        lin = np.einsum("af,bsfc->basc", feat, normal(3, 8, 16, ATOM_C, std=0.25)).astype(np.float32)
        am = np.empty_like(lin)  # [3][A][8][128]
        for s in range(8):
            if s in (0, 2, 4):  # scales: sigmoid as AF3's adaLN
                am[:, :, s] = sig(lin[:, :, s])
            elif s in (6, 7):  # gates, stored post-sigmoid
                am[:, :, s] = sig(lin[:, :, s] - 2.0)
            else:
                am[:, :, s] = lin[:, :, s]
        put(side + "_AMODS", am.astype(np.float32))
        put(side + "_APL", pair_logits())
        put(side + "_WQG", lecun_bf(3, 2 * ATOM_C, ATOM_C))
        put(side + "_BQ", normal(3, ATOM_C, std=0.1))
        put(side + "_WKV", lecun_bf(3, 2 * ATOM_C, ATOM_C))
        put(side + "_WO", lecun_bf(3, ATOM_C, ATOM_C))
        put(side + "_W1", lecun_bf(3, (6 if flags & F_ATOB else 4) * ATOM_C, ATOM_C))
        put(side + "_W2", lecun_bf(3, ATOM_C, 2 * ATOM_C))

    # variant-only inputs: present because the arity is fixed, never read with flags = 0
    put("ROPE", np.zeros((A, 32), dtype=np.float32))
    if flags & F_QKNORM:  # rows: q scale, q offset, k scale, k offset; drawn only for the variant
        def qkn(n, c):
            t = normal(n, 4, c, std=0.2)
            t[:, 0::2] += 1.0
            return t
        put("TQKN", qkn(nb, TOK_C)), put("EQKN", qkn(3, ATOM_C)), put("DQKN", qkn(3, ATOM_C))
    else:
        put("TQKN", np.zeros((nb, 4, TOK_C), dtype=np.float32))
        put("EQKN", np.zeros((3, 4, ATOM_C), dtype=np.float32))
        put("DQKN", np.zeros((3, 4, ATOM_C), dtype=np.float32))
    if flags & F_CHIRAL:
        # one chirality centre on every second token: its first four atoms, an ideal improper
        # dihedral of +-0.6 rad (every fifth centre 0 = switched off); CSR from slot to (centre, role)
        centres = np.arange(0, N, 2)
        chir_c = (centres[:, None] * SLOTS + np.arange(4)[None, :]).astype(np.int32)
        chir_a = (0.6 * np.where(np.arange(len(centres)) % 2, 1.0, -1.0)).astype(np.float32)
        chir_a[::5] = 0.0
        edges = [[] for _ in range(N * SLOTS)]
        for ci, row in enumerate(chir_c):
            for role, slot in enumerate(row):
                edges[slot].append(ci * 4 + role)
        ptr = np.zeros(N * SLOTS + 1, dtype=np.int32)
        ptr[1:] = np.cumsum([len(e) for e in edges])
        put("CHIR_W", normal(3, ATOM_C, std=0.3))
        put("CHIR_C", chir_c)
        put("CHIR_A", chir_a)
        put("CHIR_PTR", ptr)
        put("CHIR_IDX", np.array([v for e in edges for v in e], dtype=np.int32))
    else:
        put("CHIR_W", np.zeros((3, ATOM_C), dtype=np.float32))
        put("CHIR_C", np.zeros((1, 4), dtype=np.int32))
        put("CHIR_A", np.zeros(1, dtype=np.float32))
        put("CHIR_PTR", np.zeros(N * SLOTS + 1, dtype=np.int32))
        put("CHIR_IDX", np.zeros(1, dtype=np.int32))

    assert all(a is not None for a in x)
    meta = dict(N=N, A=A, NS=NS, S=samples, steps=steps, nb=nb, cs=cs, seed=seed)
    return x, meta


def noisy_positions(meta, t, seed=1):
    """A host XN for one denoiser call at noise level t: [S][N*24][3], zero on empty slots."""
    rng = np.random.default_rng(seed)
    S, N = meta["S"], meta["N"]
    return (rng.standard_normal((S, N * SLOTS, 3), dtype=np.float32) * np.float32(np.hypot(t, 10.0))).astype(np.float32)


def flops_per_eval(N, A, S, nb=24, cs=384, tw1=3072, aw1=512, nk=128):
    """Algorithmic FLOPs (2 per multiply-add; padding and the hi+lo split not counted)."""
    f_tok = nb * (2 * N * 768 * (3072 + 768 + tw1 + 1536) + 4 * N * N * 768)
    f_atom = 6 * (2 * A * 128 * (512 + 128 + aw1 + 256) + 4 * A * nk * 128)
    f_glue = 2 * A * 128 * 768 + 2 * N * 768 * 128 + 4 * A * 3 * 128
    f_cond = 2 * N * cs * (nb * 6 * 768) + 2 * (2 * N * cs * 4 * cs + 2 * N * 2 * cs * cs) + 2 * N * cs * 768 + 2 * 256 * cs
    return f_tok + f_atom + f_glue + f_cond / S


def pad_to_bucket(x, meta, n_bucket, ns_bucket, poison=False):
    """The same inputs laid out for a larger shape bucket (n_bucket tokens, ns_bucket subsets): every
    token- or atom-indexed input grows to the bucket's extent with masks 0 and index maps -1 in the
    padding. With poison=True the floating-point padding that must never influence a result (pair
    representation, single conditioning, atom conditioning) is NaN instead of 0."""
    N, A, NS = meta["N"], meta["A"], meta["NS"]
    Ab = ns_bucket * SUBSET
    assert n_bucket >= N and ns_bucket >= NS
    bad = np.float32(np.nan) if poison else np.float32(0)
    bad_bf = np.uint16(0x7FC0) if poison else np.uint16(0)
    out = [a for a in x]

    def grow(name, axis_sizes, fill):
        a = x[IN[name]]
        shape = list(a.shape)
        for ax, size in axis_sizes.items():
            shape[ax] = size
        b = np.full(shape, fill, dtype=a.dtype)
        b[tuple(slice(0, n) for n in a.shape)] = a
        out[IN[name]] = np.ascontiguousarray(b)

    grow("SC_BASE", {0: n_bucket}, bad)
    grow("PC", {0: n_bucket, 1: n_bucket}, bad_bf)
    grow("PCS", {0: n_bucket, 1: n_bucket}, bad)
    grow("TMASK", {0: n_bucket}, 0)
    grow("SCQ", {0: Ab}, bad)
    grow("QMASK", {0: Ab}, 0)
    grow("KMASK", {0: ns_bucket}, 0)
    grow("Q2K", {0: ns_bucket}, -1)
    grow("TOK2Q", {0: Ab}, -1)
    grow("Q2TA", {0: n_bucket * SLOTS}, -1)
    grow("ATOM_MASK", {0: n_bucket * SLOTS}, 0)
    grow("TAM", {0: n_bucket * SLOTS}, 0)
    grow("ROPE", {0: Ab}, 0)
    grow("CHIR_PTR", {0: n_bucket * SLOTS + 1}, 0)
    for side in ("ENC", "DEC"):
        grow(side + "_AMODS", {1: Ab}, bad)
        apl = x[IN[side + "_APL"]]
        b = np.full((3, ns_bucket) + apl.shape[2:], bad, dtype=np.float32)
        b[:, :NS] = apl
        out[IN[side + "_APL"]] = np.ascontiguousarray(b)
    m = dict(meta, N=n_bucket, A=Ab, NS=ns_bucket, real_N=N, real_NS=NS)
    return out, m


def masked_bucket_case(n_token=48, samples=2, steps=8, n_bucket=64, ns_bucket=16, absent_atoms=5, absent_tokens=2, seed=0):
    """A fold whose real extents are smaller than its shape bucket and are told by masks alone (the
    operator's ext[2] = 0: "run the bucket's extents", src/diffusion/host.cuh:223-229): the padding has
    masks 0 and index maps -1, the last real subset is partly filled (its last `absent_atoms` atom rows
    carry QMASK 0 and belong to no slot), the last `absent_tokens` real tokens are masked (TMASK 0, no
    atoms that count) and the extra pair logits PLX are present (bf16 [Nb][Nb], small values)."""
    x, meta = make_inputs(n_token, samples=samples, steps=steps, seed=seed)
    x, meta = pad_to_bucket(x, meta, n_bucket, ns_bucket)
    x = [a.copy() for a in x]
    A = meta["real_NS"] * SUBSET
    tok2q, q2ta, q2k = x[IN["TOK2Q"]], x[IN["Q2TA"]], x[IN["Q2K"]]
    gone = list(range(A - absent_atoms, A))  # the tail of the last real subset
    for n in range(n_token - absent_tokens, n_token):  # and every atom of the masked tokens
        gone += [int(a) for a in q2ta[n * SLOTS:(n + 1) * SLOTS] if a >= 0]
        x[IN["TMASK"]][n] = 0
    for a in sorted(set(gone)):
        slot = int(tok2q[a])
        if slot >= 0:
            q2ta[slot] = -1
            x[IN["ATOM_MASK"]][slot] = 0
            x[IN["TAM"]][slot] = 0
        tok2q[a] = -1
        x[IN["QMASK"]][a] = 0
        hit = q2k == a
        q2k[hit] = -1
        x[IN["KMASK"]][hit] = 0
    rng = np.random.default_rng(seed + 77)
    x[IN["PLX"]] = to_bf16((0.5 * rng.standard_normal((n_bucket, n_bucket))).astype(np.float32))
    return x, meta

// The phase schedule of the persistent sampler kernel: every step of every sample in one
// cooperative launch, one CTA per SM. Phases are separated by a grid-wide barrier built on one
// monotonic counter in global memory (release add, acquire spin, bounded).
//
// `next()` ends a phase of the reference's schedule (src/diffusion/sampler.cuh:99-230), so a debug
// run with dbg_stop = k stops at the same point in this library, in the reference and in the CPU
// oracle; `sub()` ends one of this implementation's extra sub-phases and does not count.
#pragma once

#include <new>

#include "attention_tc.cuh"
#include "positions.cuh"

namespace cck {

// phase kinds of the per-kind timing record (mk_run's `timing`): wall ns and count per kind
#define CCK_KINDS(X)                                                                               \
    X(PAIR) X(AUG) X(POS) X(INIT) X(A_LN) X(A_PROJ) X(A_ATTN) X(A_WO) X(A_LNT) X(A_W1) X(A_W2) X(A_TAIL) \
    X(AGG_GEMM) X(AGG_GATHER) X(T_ADALN) X(T_QKVG) X(T_ATTN) X(T_WO) X(T_GLU) X(T_W2) X(T_OUT) X(DEC_GLUE)
#define CCK_ENUM(name) K_##name,
enum Kind { CCK_KINDS(CCK_ENUM) kKinds };
#undef CCK_ENUM

struct Run {
    int phase = 0;        // phases of the reference's schedule finished so far
    unsigned int syncs = 0; // grid barriers passed
    bool live = true;
    unsigned long long t0 = 0; // end of the previous phase, ns
    Pipe pipe;
    TcPipe tp;
    Deal d;
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- grid barrier
__device__ __noinline__ void grid_barrier(const KP& p, Run& r, int kind) {
    fence_async_global(); // this thread's global writes, for TMA reads of other CTAs in later phases
    __syncthreads();
    if (threadIdx.x == 0) {
        SmemCtl* sc = smem_ctl();
#if CCK_STAGE_REC
        sc->stamp[5] = stage_now();
#endif
        if (sc->abort && p.ctl->status == ST_OK) {
            p.ctl->status = ST_PIPE_TIMEOUT;
            p.ctl->where = r.syncs;
        }
        const unsigned int target = (r.syncs + 1) * gridDim.x;
        red_release_add(&p.ctl->barrier, 1u);
        const long long t0 = clock64();
        while (ld_acquire(&p.ctl->barrier) < target) {
            if (clock64() - t0 > kWaitCycles) {
                if (atomicCAS(&p.ctl->status, ST_OK, ST_BARRIER_TIMEOUT) == ST_OK) {
                    p.ctl->where = r.syncs;
                }
                sc->abort = 1;
                break;
            }
            __nanosleep(20);
        }
#if CCK_STAGE_REC
        {
            const unsigned long long t = stage_now();
            if (sc->phase_t0) {
                for (int i = 0; i < 14; i++) {
                    if (i != 6 && i != 7 && sc->stamp[i] >= sc->phase_t0) {
                        atomicAdd(&g_stage_rec[kind][i], sc->stamp[i] - sc->phase_t0);
                    }
                }
                atomicAdd(&g_stage_rec[kind][6], t - sc->phase_t0);
                atomicAdd(&g_stage_rec[kind][7], 1ull);
            }
            for (int i = 0; i < 16; i++) {
                sc->stamp[i] = 0;
            }
            sc->phase_t0 = t;
        }
#endif
    }
    r.syncs++;
    if (p.timing && blockIdx.x == 0 && threadIdx.x == 0) {
        const unsigned long long t = now_ns();
        if (r.t0) {
            p.timing[2 * kind] += t - r.t0;
            p.timing[2 * kind + 1] += 1;
        }
        r.t0 = t;
    }
    __syncthreads();
#if CCK_STAGE_REC
    if (threadIdx.x == 0) {
        smem_ctl()->stamp[11] = stage_now();
    }
#endif
    fence_async_global();
#if CCK_STAGE_REC
    if (threadIdx.x == 0) {
        smem_ctl()->stamp[8] = stage_now();
    }
#endif
    r.d.start = 0;
}
// a sub-phase boundary of this implementation
__device__ __forceinline__ void sub(const KP& p, Run& r, int kind) {
    if (r.live) {
        grid_barrier(p, r, kind);
    }
}
// a phase boundary of the reference's schedule
__device__ __forceinline__ void next(const KP& p, Run& r, int kind) {
    if (!r.live) {
        return;
    }
    grid_barrier(p, r, kind);
    r.live = !(p.dbg_stop > 0 && ++r.phase >= p.dbg_stop);
    r.d.live = r.live;
}

// ---- GEMM descriptors (which GEMM feeds which buffer: reference src/diffusion/host.cuh:151-215)
__device__ inline GemmDesc make_gemm(const KP& p, int map_a, int map_b, int b_row0, int m, int n, int k, int epi,
                                     void* out, int ldo) {
    GemmDesc g{};
    g.map_a = map_a, g.map_b = map_b, g.b_row0 = b_row0, g.m = m, g.n = n, g.k = k, g.bn = p.bn[map_b];
    g.epi = epi, g.out = out, g.ldo = ldo;
    g.sig_from = n, g.bias_cols = n, g.period = 1;
    return g;
}
__device__ inline GemmDesc gemm_st_w1(const KP& p, int i) {
    return make_gemm(p, TM_A_SCT, i ? TM_B_ST1_W1 : TM_B_ST0_W1, 0, p.N, 4 * p.cs, p.cs, EPI_GLU, p.buf.sch, 2 * p.cs);
}
__device__ inline GemmDesc gemm_st_w2(const KP& p, int i) {
    return make_gemm(p, TM_A_SCH, i ? TM_B_ST1_W2 : TM_B_ST0_W2, 0, p.N, p.cs, 2 * p.cs, EPI_SCRES, p.buf.sc, p.cs);
}
__device__ inline GemmDesc gemm_mods(const KP& p, int part) {
    const int slots = part ? kTokModSlots - kTokMods1 : kTokMods1;
    GemmDesc g = make_gemm(p, part ? TM_A_SCBF : TM_A_SCLN0, part ? TM_B_WM2 : TM_B_WM1, 0, p.N, p.nb * slots * kTokC,
                           p.cs, EPI_MODS, p.buf.mods, kTokC);
    g.bias = part ? p.tw.bm2 : p.tw.bm1;
    g.slots = slots, g.slot0 = part ? kTokMods1 : 0, g.period = p.N;
    g.sig_slots = part ? (1 << TM_ATTN_GATE) | (1 << TM_TRANS_GATE) : (1 << TM_ATTN_SCALE) | (1 << TM_TRANS_SCALE);
    return g;
}
__device__ inline GemmDesc gemm_embed(const KP& p) {
    GemmDesc g = make_gemm(p, TM_A_SCLN0, TM_B_WSE, 0, p.N, kTokC, p.cs, EPI_F32, p.buf.se, kTokC);
    g.bias = p.tw.se_b;
    return g;
}
// relu(abf @ WAGGRᵀ) per atom row; the token gather follows in aggr_gather
__device__ inline GemmDesc gemm_aggr(const KP& p) {
    GemmDesc g = make_gemm(p, TM_A_ABF, TM_B_WAGGR, 0, p.S * p.A, kTokC, kAtomC, EPI_F32, p.buf.agt, kTokC);
    g.relu = 1;
    return g;
}
__device__ inline GemmDesc gemm_broadcast(const KP& p) {
    GemmDesc g = make_gemm(p, TM_A_TX, TM_B_WTB, 0, p.S * p.N, kAtomC, kTokC, EPI_F32, p.buf.tb, kAtomC);
    g.bias = p.tw.tb_b;
    return g;
}
enum TokGemm { TG_QKVG, TG_WO, TG_W1, TG_W2 };
__device__ inline GemmDesc gemm_tok(const KP& p, int b, int which) {
    const int rt = p.S * p.N;
    GemmDesc g;
    switch (which) {
    case TG_QKVG:
        g = make_gemm(p, TM_A_TX, TM_B_WQKVG, b * kQKVG, rt, kQKVG, kTokC, EPI_BF16, p.buf.qkvg, kQKVG);
        g.bias = p.tw.bq + b * kTokC, g.bias_cols = kTokC, g.sig_from = 3 * kTokC;
        g.vt = p.buf.vt, g.np = p.npb, g.period = p.N;
        break;
    case TG_WO:
        g = make_gemm(p, TM_A_TO, TM_B_WO, b * kTokC, rt, kTokC, kTokC, EPI_RESID, p.buf.act, kTokC);
        g.gate = tok_mods(p, b, TM_ATTN_GATE), g.ldg = kTokC, g.period = p.N;
        break;
    case TG_W1:
        g = make_gemm(p, TM_A_TX, TM_B_W1, b * p.tw1, rt, p.tw1, kTokC, EPI_GLU, p.buf.tc, kTokHidden);
        break;
    default:
        g = make_gemm(p, TM_A_TC, TM_B_W2, b * kTokC, rt, kTokC, kTokHidden, EPI_RESID, p.buf.act, kTokC);
        g.gate = tok_mods(p, b, TM_TRANS_GATE), g.ldg = kTokC, g.period = p.N, g.rowmask = p.tw.tmask;
    }
    return g;
}
// one-time pair logits of all blocks: row tiles are (query q, 128 keys) read straight out of PC
// (row q·Nb + k), columns the nb·16 tables
__device__ inline GemmDesc gemm_pair(const KP& p) {
    const int ktiles = cdiv(p.N, kBM);
    GemmDesc g = make_gemm(p, TM_A_PC, TM_B_PLW, 0, p.N * ktiles * kBM, p.nb * kPairHeads, p.plc, EPI_PAIR, p.buf.plg, 0);
    g.np = p.npb, g.ldn = p.Nb, g.ktiles = ktiles, g.nreal = p.N, g.npreal = p.np;
    g.pcs = p.tw.pcs, g.plws = p.tw.plws, g.plb = p.tw.plb, g.tmask = p.tw.tmask;
    g.plx = p.plx ? p.tw.plx : nullptr;
    return g;
}
enum AtomGemm { AG_QG, AG_KV, AG_WO, AG_W1, AG_W2 };
__device__ inline GemmDesc gemm_atom(const KP& p, int side, int b, int which) {
    const AtomW& w = side ? p.dec : p.enc;
    const int ra = p.S * p.A, m0 = side ? TM_B_DEC_WQG : TM_B_ENC_WQG;
    const float* am = w.amods + size_t(b) * p.NSb * kSubset * kAtomModSlots * kAtomC;
    GemmDesc g;
    switch (which) {
    case AG_QG:
        g = make_gemm(p, TM_A_AXQ, m0 + 0, b * 2 * kAtomC, ra, 2 * kAtomC, kAtomC, EPI_BF16, p.buf.aqg, 2 * kAtomC);
        g.bias = w.bq + b * kAtomC, g.bias_cols = kAtomC, g.sig_from = kAtomC;
        break;
    case AG_KV:
        g = make_gemm(p, TM_A_AXK, m0 + 1, b * 2 * kAtomC, ra, 2 * kAtomC, kAtomC, EPI_BF16, p.buf.akv, 2 * kAtomC);
        break;
    case AG_WO: // qa += am6 ⊙ (ao @ WOᵀ)
        g = make_gemm(p, TM_A_AO, m0 + 2, b * kAtomC, ra, kAtomC, kAtomC, EPI_RESID, p.buf.qa, kAtomC);
        g.gate = am + AM_ATTN_GATE * kAtomC, g.gate_f32 = 1, g.ldg = kAtomModSlots * kAtomC, g.period = p.A;
        break;
    case AG_W1: // [hi | lo] inputs against the same W1 columns twice
        g = make_gemm(p, TM_A_AXHL, m0 + 3, b * p.aw1, ra, p.aw1, 2 * kAtomC, EPI_GLU, p.buf.aca, kAtomHidden);
        g.b_kwrap = kAtomC;
        break;
    default: // qa += QMASK · am7 ⊙ (c @ W2ᵀ)
        g = make_gemm(p, TM_A_ACA, m0 + 4, b * kAtomC, ra, kAtomC, kAtomHidden, EPI_RESID, p.buf.qa, kAtomC);
        g.gate = am + AM_T_GATE * kAtomC, g.gate_f32 = 1, g.ldg = kAtomModSlots * kAtomC, g.period = p.A;
        g.rowmask = p.geo.qmask;
    }
    return g;
}

template <int N> __device__ __forceinline__ void run_gemms(const Launch& L, Run& r, const GemmDesc (&list)[N]) {
    if (r.live) {
        gemm_phase(L, r.pipe, r.d, list, N);
    }
}

// What the pair-logit GEMM does not write but attention may read: VT's key pads (P is exactly zero
// there, the value only has to be finite), the rows of QKVG just past the last sample (a key tile
// of the last sample reaches into them), and PLG's query rows between N and the padded extent.
__device__ void pair_fill_pads(const KP& p, Deal& d) {
    const int pad = p.np - p.N;
    const size_t tid = size_t(blockIdx.x) * kThreads + threadIdx.x, nth = size_t(gridDim.x) * kThreads;
    if (pad > 0) {
        const size_t v = size_t(p.S) * kTokC * pad;
        for (size_t i = tid; i < v; i += nth) {
            p.buf.vt[(i / pad) * p.npb + p.N + i % pad] = 0;
        }
        const size_t tables = size_t(p.nb) * kPairHeads, m = tables * pad * p.np;
        for (size_t i = tid; i < m; i += nth) {
            const size_t tb = i / (size_t(pad) * p.np), rest = i % (size_t(pad) * p.np);
            p.buf.plg[(tb * p.npb + p.N + rest / p.np) * p.npb + rest % p.np] = 0;
        }
    }
    const size_t row0 = size_t(p.S) * p.N, row1 = min(size_t(p.S) * p.Nb, row0 + kTcKeys);
    uint4* z = reinterpret_cast<uint4*>(p.buf.qkvg + row0 * kQKVG);
    for (size_t i = tid; i < (row1 - row0) * kQKVG / 8; i += nth) {
        z[i] = make_uint4(0, 0, 0, 0);
    }
    (void)d;
}

// ---- the atom block: adaLN + projections | attention | out-projection, transition, tails
// (reference phases A_QKV, A_ATTN, A_GLU: src/diffusion/sampler.cuh:87-97)
enum Tail { TAIL_NONE, TAIL_SKIP, TAIL_UPDATE };

__device__ void atom_proj(const Launch& L, Run& r, int side, int b) {
    const KP& p = kp();
    if (r.live) {
        atom_ln_qk(p, r.d, side ? p.dec : p.enc, b);
    }
    sub(p, r, K_A_LN);
    const GemmDesc g[2] = {gemm_atom(p, side, b, AG_QG), gemm_atom(p, side, b, AG_KV)};
    run_gemms(L, r, g);
}
// `extra` rides in the first sub-phase (the conditioning's st_w2 during the encoder); returns the
// kind of the last sub-phase, which the caller ends
__device__ int atom_mlp(const Launch& L, Run& r, int side, int b, int tail, const GemmDesc* extra) {
    const KP& p = kp();
    const AtomW& w = side ? p.dec : p.enc;
    if (extra) {
        const GemmDesc g[2] = {*extra, gemm_atom(p, side, b, AG_WO)};
        run_gemms(L, r, g);
    } else {
        const GemmDesc g[1] = {gemm_atom(p, side, b, AG_WO)};
        run_gemms(L, r, g);
    }
    sub(p, r, K_A_WO);
    if (r.live) {
        atom_ln_t(p, r.d, w, b);
    }
    sub(p, r, K_A_LNT);
    {
        const GemmDesc g[1] = {gemm_atom(p, side, b, AG_W1)};
        run_gemms(L, r, g);
    }
    sub(p, r, K_A_W1);
    {
        const GemmDesc g[1] = {gemm_atom(p, side, b, AG_W2)};
        run_gemms(L, r, g);
    }
    if (tail != TAIL_NONE) {
        sub(p, r, K_A_W2);
        if (r.live) {
            if (tail == TAIL_SKIP) {
                atom_tail_skip(p, r.d);
            } else {
                atom_tail_update(p, r.d);
            }
        }
        return K_A_TAIL;
    }
    return K_A_W2;
}

// reference: src/diffusion/sampler.cuh:99-134 (flags = 0, pair logits resident)
__device__ void token_block(const Launch& L, Run& r, int b) {
    const KP& p = kp();
    if (r.live) {
        token_adaln(p, r.d, b, TM_ATTN_SCALE);
    }
    next(p, r, K_T_ADALN);
    {
        const GemmDesc g[1] = {gemm_tok(p, b, TG_QKVG)};
        run_gemms(L, r, g);
    }
    next(p, r, K_T_QKVG);
    if (r.live) {
        if (p.attn_warp) {
            token_attention(p, r.d, b);
        } else {
            r.d.advance(token_attention_tc(L, r.d, r.tp, b));
        }
    }
    next(p, r, K_T_ATTN);
    {
        const GemmDesc g[1] = {gemm_tok(p, b, TG_WO)};
        run_gemms(L, r, g);
    }
    next(p, r, K_T_WO);
    if (r.live) {
        token_adaln(p, r.d, b, TM_TRANS_SCALE);
    }
    next(p, r, K_T_ADALN);
    {
        const GemmDesc g[1] = {gemm_tok(p, b, TG_W1)};
        run_gemms(L, r, g);
    }
    next(p, r, K_T_GLU);
    {
        const GemmDesc g[1] = {gemm_tok(p, b, TG_W2)};
        run_gemms(L, r, g);
    }
    next(p, r, K_T_W2);
}

// one denoiser call at noise level t on XN, ending with UPD (reference: src/diffusion/sampler.cuh:137-182)
__device__ void denoise(const Launch& L, Run& r, float t) {
    const KP& p = kp();
    if (r.live) {
        noise_vector(p, r.d, t);
        atom_init(p, r.d, t);
    }
    next(p, r, K_INIT);
    for (int b = 0; b < kAtomBlocks; b++) {
        if (r.live) {
            if (b < 2) {
                sc_layernorm(p, r.d, b, b == 0);
            } else {
                sc_prep(p, r.d);
            }
        }
        atom_proj(L, r, 0, b);
        next(p, r, K_A_PROJ);
        if (b < 2) {
            const GemmDesc g[1] = {gemm_st_w1(p, b)};
            run_gemms(L, r, g);
        } else {
            const GemmDesc g[3] = {gemm_mods(p, 0), gemm_mods(p, 1), gemm_embed(p)};
            run_gemms(L, r, g);
        }
        if (r.live) {
            __syncthreads(); // the GEMM roles rejoin before the CTA restages shared memory
            atom_attention(p, r.d, p.enc, b);
        }
        next(p, r, K_A_ATTN);
        int kind;
        if (b < 2) {
            const GemmDesc w2 = gemm_st_w2(p, b);
            kind = atom_mlp(L, r, 0, b, TAIL_NONE, &w2);
        } else {
            kind = atom_mlp(L, r, 0, b, TAIL_SKIP, nullptr);
        }
        next(p, r, kind);
    }
    {
        const GemmDesc g[1] = {gemm_aggr(p)};
        run_gemms(L, r, g);
    }
    sub(p, r, K_AGG_GEMM);
    if (r.live) {
        aggr_gather(p, r.d);
    }
    next(p, r, K_AGG_GATHER);
    for (int b = 0; b < p.nb; b++) {
        token_block(L, r, b);
    }
    if (r.live) {
        token_final_ln(p, r.d);
    }
    next(p, r, K_T_OUT);
    {
        const GemmDesc g[1] = {gemm_broadcast(p)};
        run_gemms(L, r, g);
    }
    next(p, r, K_T_OUT);
    if (r.live) {
        decoder_init(p, r.d);
    }
    next(p, r, K_DEC_GLUE);
    for (int b = 0; b < kAtomBlocks; b++) {
        atom_proj(L, r, 1, b);
        next(p, r, K_A_PROJ);
        if (r.live) {
            atom_attention(p, r.d, p.dec, b);
        }
        next(p, r, K_A_ATTN);
        const int kind = atom_mlp(L, r, 1, b, b + 1 < kAtomBlocks ? TAIL_NONE : TAIL_UPDATE, nullptr);
        next(p, r, kind);
    }
}

__device__ void build_pairs(const Launch& L, Run& r) {
    if (r.live) {
        pair_fill_pads(kp(), r.d);
    }
    const GemmDesc g[1] = {gemm_pair(kp())};
    run_gemms(L, r, g);
}

// reference: src/diffusion/sampler.cuh:184-217 (Euler path)
__device__ void sample(const Launch& L, Run& r) {
    const KP& p = kp();
    positions_init(p, r.d);
    build_pairs(L, r);
    next(p, r, K_PAIR);
    for (int step = 1; step <= p.nsteps && r.live; step++) {
        const StepNoise sn = step_noise(p, step);
        positions_centre(p, r.d);
        next(p, r, K_AUG);
        if (r.live) {
            positions_augment(p, r.d, step);
        }
        next(p, r, K_AUG);
        denoise(L, r, sn.t_hat);
        if (r.live) {
            positions_update(p, r.d, step, false);
        }
        next(p, r, K_POS);
    }
    if (r.live) {
        positions_output(p, r.d);
    }
}

// mode 1: one denoiser call on the caller's XN at t; denoised positions to OUT
// (reference: src/diffusion/sampler.cuh:219-230)
__device__ void denoise_once(const Launch& L, Run& r) {
    const KP& p = kp();
    build_pairs(L, r);
    next(p, r, K_PAIR);
    denoise(L, r, p.t);
    if (r.live) {
        positions_update(p, r.d, 0, true);
    }
    next(p, r, K_POS);
}

} // namespace cck

extern "C" __global__ void __launch_bounds__(cck::kThreads, 1) cck_sampler_kernel(const __grid_constant__ cck::Launch L) {
    using namespace cck;
    // the CTA's parameter block: the kernel parameter with the real extents of this call, which
    // arrive in device memory (ext = {N, NS, exact, seed_lo, seed_hi}) and are clamped to the bucket
    {
        uint32_t* dst = reinterpret_cast<uint32_t*>(smem_base() + kKpOff);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&L.kp);
        for (int i = threadIdx.x; i < int(sizeof(KP) / 4); i += kThreads) {
            dst[i] = src[i];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            KP& w = *reinterpret_cast<KP*>(dst);
            if (w.ext && w.ext[2]) {
                w.N = max(1, min(w.ext[0], w.Nb)), w.NS = max(1, min(w.ext[1], w.NSb));
            }
            w.A = w.NS * kSubset, w.np = cdiv(w.N, kTcKeys) * kTcKeys, w.chunks = cdiv(w.N * kSlots, kChunk);
        }
        __syncthreads();
    }
    const KP& p = kp();
    gemm_init();
    attn_tc_init();
#if CCK_STAGE_REC
    if (threadIdx.x == 0) {
        for (int i = 0; i < 16; i++) {
            smem_ctl()->stamp[i] = 0;
        }
        smem_ctl()->phase_t0 = 0;
    }
#endif
    __syncthreads();
    // The schedule state of each thread lives in shared memory, not on its stack: the acquire of
    // every grid barrier empties L1, and state kept in local memory would then cost an L2 round
    // trip per touch right at the start of every phase.
    static_assert(sizeof(Run) <= kRunSlot, "Run outgrew its shared-memory slot");
    Run& r = *new (smem_base() + kRunOff + threadIdx.x * kRunSlot) Run();
    if (kp().mode == 0) {
        sample(L, r);
    } else {
        denoise_once(L, r);
    }
    gemm_fini();
}

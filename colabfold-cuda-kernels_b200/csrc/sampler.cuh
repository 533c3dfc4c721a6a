// The phase schedule of the persistent sampler kernel: every step of every sample in one
// cooperative launch, one CTA per SM. Phases are separated by a grid-wide barrier built on one
// monotonic counter in global memory (release add, acquire spin, bounded).
//
// The schedule itself is data: the host writes the phase program (host.cuh: make_program), this
// file interprets it. An operation marked END_PHASE ends a phase of the reference's schedule
// (src/diffusion/sampler.cuh:99-230), so a debug run with dbg_stop = k stops at the same point in
// this library, in the reference and in the CPU oracle; END_SUB ends one of this implementation's
// extra sub-phases and does not count.
#pragma once

#include <new>

#include "attention_tc.cuh"
#include "positions.cuh"

namespace cck {

struct Run {
    unsigned short phase = 0; // phases of the reference's schedule finished so far
    unsigned char pc = 0;     // the operation of the program being run
    unsigned char blk = 0;    // token block of the loop
    unsigned int syncs = 0;   // grid barriers passed
    unsigned short step = 0;  // sampling step
    unsigned char ret = 0;    // where the denoiser subroutine returns to
    unsigned char second = 0; // the subroutine runs at σ (Heun's second call)
    Pipe pipe;
    Deal d;                   // the work dealing's rotation inside a phase
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- the program's control flow: from (pc, blk, step, ret, second) to the next operation that does
// work (or FN_END). Used by the interpreter, and without side effects by the barrier's look-ahead.
struct Flow {
    int pc, blk, step, ret, second;
};
__device__ __forceinline__ Op flow_next(const Program& prog, const KP& p, Flow& f) {
    for (;;) {
        const Op op = prog.ops[f.pc];
        if (op.fn == FN_BLOCK_NEXT) {
            f.blk = f.blk + 1 < p.nb ? f.blk + 1 : 0;
            f.pc = f.blk ? op.a0 : f.pc + 1;
        } else if (op.fn == FN_STEP_NEXT) {
            f.step++;
            f.pc = f.step <= p.nsteps ? op.a0 : f.pc + 1;
        } else if (op.fn == FN_CALL) {
            f.ret = f.pc + 1, f.second = op.b, f.pc = op.a0;
        } else if (op.fn == FN_RET) {
            f.pc = f.ret;
        } else {
            return op;
        }
    }
}

// ---- grid barrier
// The schedule state of the calling thread (shared memory)
__device__ __forceinline__ Run& run_state() {
    return *reinterpret_cast<Run*>(smem_base() + kRunOff + threadIdx.x * kRunSlot);
}
// Ends a phase (end_kind: OpEnd in the low two bits, the timing kind above). Returns true when a debug
// run has reached its last phase. Takes and returns next to nothing, so that the caller holds no
// registers across it.
__device__ __noinline__ bool grid_barrier(const Launch& L, int end_kind) {
    const KP& p = kp();
    Run& r = run_state();
    const int kind = end_kind >> 2;
    const bool stop = (end_kind & 3) == END_PHASE && p.dbg_stop > 0 && r.phase + 1 >= p.dbg_stop;
    fence_async_global(); // this thread's global writes, for TMA reads of other CTAs in later phases
    __syncthreads();
    // Thread 0 waits for the grid; its warp then releases the CTA through a named barrier (the warp
    // arrives as a whole and does not wait: a warp-level barrier instruction counts 32 arrivals
    // however many of its lanes run it, so the warp must not be split between arrive and sync),
    // after which thread 0 runs the next GEMM's TMA role while the others find their way there.
    int gemm_id = -1, gemm_b = 0;
    bool open = true;
    if (threadIdx.x == 0) {
        SmemCtl* sc = smem_ctl();
#if CCK_STAGE_REC
        sc->stamp[5] = stage_now();
#endif
        if (sc->abort) { // a wait of this CTA gave up in the phase that ends here
            fail_launch(ST_PIPE_TIMEOUT, r.syncs);
        }
        const unsigned int target = (r.syncs + 1) * gridDim.x + (unsigned int)p.barrier_extra;
        CCK_TRACE_ONE(6, 0x84, kind);
#if CCK_TRACE
        const long long tw0_ = clock64();
#endif
        red_release_add(&p.ctl->barrier, 1u);
        // while the arrival travels: is the next operation a GEMM? (the program's control
        // operations followed without their side effects)
        if (!stop) {
            const Program& prog = *reinterpret_cast<const Program*>(smem_base() + kProgOff);
            Flow f{r.pc, r.blk, r.step, r.ret, r.second};
            const Op op = flow_next(prog, p, f);
            if (op.fn == FN_GEMM) { // (a GEMM that waits for other units never follows a barrier: nothing to wait for here)
                gemm_id = op.a0, gemm_b = op.b == kLoopB ? f.blk : op.b;
            }
        }
        const long long t0 = clock64();
        for (;;) {
            const unsigned int v = ld_acquire(&p.ctl->barrier);
            if (v & kBarrierPoison) { // some CTA has recorded a failure: nobody waits for anybody any more
                sc->abort = 1, sc->quit = 1;
                open = false;
                break;
            }
            if (v >= target) {
                break;
            }
            if (clock64() - t0 > wait_limit()) {
                fail_launch(ST_BARRIER_TIMEOUT, r.syncs);
                sc->abort = 1, sc->quit = 1;
                open = false;
                break;
            }
            __nanosleep(20);
        }
        CCK_TRACE_ONE(6, 0x86, kind);
#if CCK_TRACE
        if (r.syncs < kBarWaitSlots) { // every CTA: how long it waited at this barrier (the last to arrive waits least)
            g_barwait[r.syncs][blockIdx.x] = (unsigned int)(clock64() - tw0_) | (unsigned int)kind << 24;
        }
#endif
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
        if (p.timing && blockIdx.x == 0) {
            const unsigned long long t = now_ns();
            if (sc->t0) {
                // accumulated in shared memory, written out when the kernel ends: a global
                // read-modify-write here would delay CTA 0, and with it the grid, in every phase
                unsigned long long* acc = reinterpret_cast<unsigned long long*>(smem_base() + kCtlOff + kTimingOff);
                acc[2 * kind] += t - sc->t0;
                acc[2 * kind + 1] += 1;
            }
            sc->t0 = t;
        }
        open = open && !sc->abort;
    }
    if (warp_id() == 0) {
        __syncwarp();
        asm volatile("barrier.cta.arrive 6, %0;" ::"n"(kThreads) : "memory");
        if (threadIdx.x == 0 && open && gemm_id >= 0) {
            fence_async_global(); // the other CTAs' writes of the phase just ended, for this thread's TMA reads
            const GemmDesc& g = gd_table()[gemm_id];
            gemm_produce(L, r.pipe, g, gemm_b, blockIdx.x, g.tiles, gridDim.x, true, 0); // the rotation starts at 0 after a barrier
        }
        __syncwarp();
    } else {
        asm volatile("barrier.cta.sync 6, %0;" ::"n"(kThreads) : "memory");
    }
    r.syncs++;
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
    r.phase += (end_kind & 3) == END_PHASE;
    return stop || smem_ctl()->quit; // (written before the named barrier that released this thread)
}

// ---- GEMM descriptors (which GEMM feeds which buffer: reference src/diffusion/host.cuh:151-215)
// The table is built once per launch (gd_build) for block 0 of every stack, with what a block adds.
static_assert(kNumGd <= kMaxGd, "the descriptor table outgrew its shared-memory slot");
__device__ inline GemmDesc make_gemm(const KP& p, int map_a, int map_b, int b_row0, int m, int n, int k, int epi,
                                     void* out, int ldo) {
    GemmDesc g{};
    g.map_a = map_a, g.map_b = map_b, g.b_row0 = b_row0, g.m = m, g.n = n, g.k = k, g.bn = p.bn[map_b];
    g.epi = epi, g.out = out, g.ldo = ldo, g.map_o = -1, g.glu_unit = 2 * kGluHalf;
    g.sig_from = n, g.bias_cols = n, g.period = 1;
    return g;
}
__device__ inline GemmDesc gemm_st_w1(const KP& p, int i) {
    GemmDesc g = make_gemm(p, TM_A_SCT, i ? TM_B_ST1_W1 : TM_B_ST0_W1, 0, p.N, 4 * p.cs, p.cs, EPI_GLU, p.buf.sch, 2 * p.cs);
    g.map_o = TM_O_SCH;
    return g;
}
__device__ inline GemmDesc gemm_st_w2(const KP& p, int i) {
    return make_gemm(p, TM_A_SCH, i ? TM_B_ST1_W2 : TM_B_ST0_W2, 0, p.N, p.cs, 2 * p.cs, EPI_SCRES, p.buf.sc, p.cs);
}
__device__ inline GemmDesc gemm_mods(const KP& p, int part) {
    const int slots = part ? kTokModSlots - kTokMods1 : kTokMods1;
    // IDSCALE: the modulations read sc itself and the scale slots stay linear (reference: src/diffusion/host.cuh:155-167)
    const bool idscale = p.flags & F_IDSCALE;
    GemmDesc g = make_gemm(p, part || idscale ? TM_A_SCBF : TM_A_SCLN0, part ? TM_B_WM2 : TM_B_WM1, 0, p.N, p.nb * slots * kTokC,
                           p.cs, EPI_MODS, p.buf.mods, kTokC);
    g.bias = part ? p.tw.bm2 : p.tw.bm1;
    g.slots = slots, g.slot0 = part ? kTokMods1 : 0, g.period = p.N, g.map_o = TM_O_MODS;
    g.sig_slots = part ? (1 << TM_ATTN_GATE) | (1 << TM_TRANS_GATE) : idscale ? 0 : (1 << TM_ATTN_SCALE) | (1 << TM_TRANS_SCALE);
    return g;
}
__device__ inline GemmDesc gemm_embed(const KP& p) {
    GemmDesc g = make_gemm(p, p.flags & F_IDSCALE ? TM_A_SCBF : TM_A_SCLN0, TM_B_WSE, 0, p.N, kTokC, p.cs, EPI_F32, p.buf.se, kTokC);
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
        g.vt = p.buf.vt, g.np = p.npb, g.period = p.N, g.map_o = TM_O_QKVG;
        break;
    case TG_WO:
        g = make_gemm(p, TM_A_TO, TM_B_WO, b * kTokC, rt, kTokC, kTokC, EPI_RESID, p.buf.act, kTokC);
        g.gate = tok_mods(p, b, TM_ATTN_GATE), g.ldg = kTokC, g.period = p.N;
        break;
    case TG_W1:
        g = make_gemm(p, p.flags & F_PARALLEL ? TM_A_TX2 : TM_A_TX, TM_B_W1, b * p.tw1, rt, p.tw1, kTokC, EPI_GLU, p.buf.tc, kTokHidden);
        g.map_o = TM_O_TC, g.glu_unit = p.tw1 / (kTokHidden / kGluHalf);
        break;
    default:
        g = make_gemm(p, TM_A_TC, TM_B_W2, b * kTokC, rt, kTokC, kTokHidden, EPI_RESID, p.buf.act, kTokC);
        g.gate = tok_mods(p, b, TM_TRANS_GATE), g.ldg = kTokC, g.period = p.N, g.rowmask = p.tw.tmask;
    }
    if (p.flow) { // blocks of 128 rows complete in order, and the units that read them start early
        const int sig = 1 + (which == TG_QKVG ? FC_QKVG : which == TG_WO ? FC_ACT1 : which == TG_W1 ? FC_TC : FC_ACT2);
        const int dep = which == TG_WO ? 1 + FC_TO : which == TG_W1 ? 1 + FC_TX : which == TG_W2 ? 1 + FC_TC : 0;
        g.fl = GF_NFAST | sig << GF_SIG_SHIFT | dep << GF_DEP_SHIFT;
    }
    return g;
}
// one-time pair logits of all blocks: row tiles are (query q, 128 keys) read straight out of PC
// (row q·Nb + k), columns the nb·16 tables
__device__ inline GemmDesc gemm_pair(const KP& p) {
    const int ktiles = cdiv(p.N, kBM);
    GemmDesc g = make_gemm(p, TM_A_PC, TM_B_PLW, 0, p.N * ktiles * kBM, p.nb * kPairHeads, p.plc, EPI_PAIR, p.buf.plg, 0);
    g.np = p.npb, g.ldn = p.Nb, g.ktiles = ktiles, g.nreal = p.N, g.npreal = p.np;
    return g;
}
__device__ inline GemmDesc gemm_atom(const KP& p, int side, int b, int which) {
    const AtomW& w = side ? p.dec : p.enc;
    const int ra = p.S * p.A, m0 = side ? TM_B_DEC_WQG : TM_B_ENC_WQG;
    const float* am = w.amods + size_t(b) * p.NSb * kSubset * kAtomModSlots * kAtomC;
    GemmDesc g;
    switch (which) {
    case AG_QG:
        g = make_gemm(p, TM_A_AXQ, m0 + 0, b * 2 * kAtomC, ra, 2 * kAtomC, kAtomC, EPI_BF16, p.buf.aqg, 2 * kAtomC);
        g.bias = w.bq + b * kAtomC, g.bias_cols = kAtomC, g.sig_from = kAtomC, g.map_o = TM_O_AQG;
        break;
    case AG_KV:
        g = make_gemm(p, TM_A_AXK, m0 + 1, b * 2 * kAtomC, ra, 2 * kAtomC, kAtomC, EPI_BF16, p.buf.akv, 2 * kAtomC);
        g.map_o = TM_O_AKV;
        break;
    case AG_WO: // qa += am6 ⊙ (ao @ WOᵀ)
        g = make_gemm(p, TM_A_AO, m0 + 2, b * kAtomC, ra, kAtomC, kAtomC, EPI_RESID, p.buf.qa, kAtomC);
        g.gate = am + AM_ATTN_GATE * kAtomC, g.gate_f32 = 1, g.ldg = kAtomModSlots * kAtomC, g.period = p.A;
        break;
    case AG_W1: // [hi | lo] inputs against the same W1 columns twice
        g = make_gemm(p, TM_A_AXHL, m0 + 3, b * p.aw1, ra, p.aw1, 2 * kAtomC, EPI_GLU, p.buf.aca, kAtomHidden);
        g.b_kwrap = kAtomC, g.map_o = TM_O_ACA, g.glu_unit = p.aw1 / (kAtomHidden / kGluHalf);
        break;
    default: // qa += QMASK · am7 ⊙ (c @ W2ᵀ)
        g = make_gemm(p, TM_A_ACA, m0 + 4, b * kAtomC, ra, kAtomC, kAtomHidden, EPI_RESID, p.buf.qa, kAtomC);
        g.gate = am + AM_T_GATE * kAtomC, g.gate_f32 = 1, g.ldg = kAtomModSlots * kAtomC, g.period = p.A;
        g.rowmask = p.geo.qmask;
    }
    return g;
}
// descriptor `id` of the table, as of block b of its stack
__device__ __noinline__ GemmDesc gd_make(const KP& p, int id, int b) {
    switch (id) {
    case GD_ST_W1_0:
    case GD_ST_W1_1:
        return gemm_st_w1(p, id - GD_ST_W1_0);
    case GD_ST_W2_0:
    case GD_ST_W2_1:
        return gemm_st_w2(p, id - GD_ST_W2_0);
    case GD_MODS_0:
    case GD_MODS_1:
        return gemm_mods(p, id - GD_MODS_0);
    case GD_EMBED:
        return gemm_embed(p);
    case GD_AGGR:
        return gemm_aggr(p);
    case GD_BROADCAST:
        return gemm_broadcast(p);
    case GD_PAIR:
        return gemm_pair(p);
    case GD_TOK_QKVG:
    case GD_TOK_WO:
    case GD_TOK_W1:
    case GD_TOK_W2:
        return gemm_tok(p, b, id - GD_TOK_QKVG);
    default:
        return gemm_atom(p, id >= GD_DEC_QG, b, (id - GD_ENC_QG) % 5);
    }
}
// thread i builds descriptor i; the difference between blocks 1 and 0 is what a block adds
__device__ __noinline__ void gd_build() {
    const KP& p = kp();
    if (threadIdx.x < kNumGd) {
        GemmDesc g = gd_make(p, threadIdx.x, 0);
        const GemmDesc g1 = gd_make(p, threadIdx.x, 1);
        g.b_step = g1.b_row0 - g.b_row0;
        g.bias_step = g.bias ? int(g1.bias - g.bias) : 0;
        g.gate_step = static_cast<const char*>(g1.gate) - static_cast<const char*>(g.gate);
        gd_finish(g);
        gd_table()[threadIdx.x] = g;
    }
    __syncthreads();
}

// What the pair-logit GEMM does not write but attention may read: VT's key pads (P is exactly zero
// there, the value only has to be finite), the rows of QKVG just past the last sample (a key tile
// of the last sample reaches into them), and PLG's query rows between N and the padded extent.
__device__ CCK_PHASE_FN void pair_fill_pads(const KP& p, Deal& d) {
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
    if (p.flow) { // the completion counters of the token blocks' chains
        for (size_t i = tid; i < size_t(kFlowCnts) * p.flow_n; i += nth) {
            p.flow_cnt[i] = 0;
        }
    }
    const size_t row0 = size_t(p.S) * p.N, row1 = min(size_t(p.S) * p.Nb, row0 + kTcKeys);
    uint4* z = reinterpret_cast<uint4*>(p.buf.qkvg + row0 * kQKVG);
    for (size_t i = tid; i < (row1 - row0) * kQKVG / 8; i += nth) {
        z[i] = make_uint4(0, 0, 0, 0);
    }
    (void)d;
}

// ---- the interpreter of the phase program
// Every function an operation can name is out of line and called from this one level, with next to
// nothing live across the call: registers of a callee come on top of what its callers hold, so a
// deep or fat call chain would push the heavy phase functions into spills.
__device__ __forceinline__ void run_gemm(const Launch& L, Run& r, Deal& d, int id, int b, unsigned int epoch) {
    const GemmDesc& g = gd_table()[id];
    const int tiles = g.tiles, tb = d.first(), ts = gridDim.x;
    const int warp = warp_id();
    if (threadIdx.x == 0) {
        CCK_STAMP(9, true);
    }
    if (warp == 0) {
        if (lane_id() == 0) {
            gemm_produce(L, r.pipe, g, b, tb, tiles, ts, false, epoch);
        }
    } else if (warp == 1) {
        if (lane_id() == 0) {
            gemm_issue(r.pipe, g, tb, tiles, ts);
        }
    } else if (warp < kAuxWarp0) {
        const uint32_t tile = r.pipe.tile;
        const CUtensorMap* mo = g.map_o >= 0 ? &L.tmap[g.map_o] : nullptr;
        switch (g.epi) {
        case EPI_BF16:
            worker_tiles<EPI_BF16>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        case EPI_F32:
            worker_tiles<EPI_F32>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        case EPI_SCRES:
            worker_tiles<EPI_SCRES>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        case EPI_MODS:
            worker_tiles<EPI_MODS>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        case EPI_GLU:
            worker_tiles<EPI_GLU>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        case EPI_RESID:
            worker_tiles<EPI_RESID>(g, mo, b, tile, tb, tiles, ts, epoch);
            break;
        default:
            worker_tiles<EPI_PAIR>(g, mo, b, tile, tb, tiles, ts, epoch);
        }
        r.pipe.tile = tile + (tiles > tb ? (tiles - tb + ts - 1) / ts : 0);
    }
    __syncwarp();
    d.advance(tiles);
}

// How many token blocks of this launch came before the current one (denoiser calls so far x blocks
// + the block): the completion counters count on through the launch and are compared with multiples of it
__device__ __forceinline__ unsigned int flow_epoch(const KP& p, const Run& r) {
    const int calls_per_step = (p.flags & F_HEUN) && !(p.flags & F_REALIGN) ? 2 : 1;
    const int calls = p.mode == 0 ? (int(r.step) - 1) * calls_per_step + r.second : 0;
    return (unsigned int)(calls * p.nb + r.blk);
}
// one operation of the program; everything it needs comes from shared memory
__device__ __forceinline__ void run_op(const Launch& L, Run& r, const Op op) {
    const KP& p = kp();
    const int b = op.b == kLoopB ? r.blk : op.b, step = r.step;
    Deal& d = r.d;
    if (threadIdx.x == 0) {
        CCK_STAMP(12, true);
    }
    switch (op.fn) {
    case FN_GEMM:
        run_gemm(L, r, d, op.a0, b, flow_epoch(p, r));
        break;
    case FN_POS_INIT:
        positions_init(p, d);
        break;
    case FN_PAIR_PADS:
        pair_fill_pads(p, d);
        break;
    case FN_POS_CENTRE:
        positions_centre(p, d);
        break;
    case FN_POS_AUGMENT:
        positions_augment(p, d, step);
        break;
    case FN_POS_UPDATE:
        positions_update(p, d, step, UPDATE_EULER);
        break;
    case FN_POS_OUT_ONCE:
        positions_update(p, d, 0, UPDATE_OUT);
        break;
    case FN_POS_HEUN1:
        positions_update(p, d, step, UPDATE_HEUN1);
        break;
    case FN_POS_HEUN2:
        positions_update(p, d, step, UPDATE_HEUN2);
        break;
    case FN_POS_MOMENTS:
        positions_moments(p, d, step);
        break;
    case FN_POS_REALIGN:
        positions_realign(p, d, step);
        break;
    case FN_POS_OUTPUT:
        positions_output(p, d);
        break;
    case FN_NOISE_INIT: {
        const float t = p.mode != 0 ? p.t : r.second ? step_noise(p, step).sigma : step_noise(p, step).t_hat;
        noise_vector(p, d, t);
        atom_init(p, d, t);
        break;
    }
    case FN_SC_LN:
        sc_layernorm(p, d, op.a0, op.a0 == 0);
        break;
    case FN_SC_PREP:
        sc_prep(p, d);
        break;
    case FN_ATOM_LN_QK:
        atom_ln_qk(p, d, op.a0 ? p.dec : p.enc, b);
        break;
    case FN_ATOM_ATTN:
        atom_attention(p, d, op.a0 ? p.dec : p.enc, b);
        break;
    case FN_ATOM_LN_T:
        atom_ln_t(p, d, op.a0 ? p.dec : p.enc, b);
        break;
    case FN_ATOM_TAIL_SKIP:
        atom_tail_skip(p, d);
        break;
    case FN_ATOM_TAIL_UPDATE:
        atom_tail_update(p, d);
        break;
    case FN_AGGR_GATHER:
        aggr_gather(p, d);
        break;
    case FN_TOK_ADALN:
        token_adaln(p, d, b, op.a0, flow_epoch(p, r));
        break;
    case FN_TOK_ADALN2:
        token_adaln2(p, d, b);
        break;
    case FN_TOK_ATTN:
        d.advance(token_attention_tc(L, d, b, flow_epoch(p, r)));
        break;
    case FN_TOK_FINAL_LN:
        token_final_ln(p, d, flow_epoch(p, r) + p.nb); // (the loop has set the block back to 0)
        break;
    case FN_DEC_INIT:
        decoder_init(p, d);
        break;
    case FN_TOK_QKNORM:
        token_qknorm(p, d, b);
        break;
    case FN_ATOM_QKNORM:
        atom_qknorm(p, d, op.a0 ? p.dec : p.enc, b);
        break;
    default: // FN_CTA_SYNC
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        CCK_STAMP(13, false);
    }
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
        // the phase program too: an operation is fetched at the start of every phase
        uint32_t* pd = reinterpret_cast<uint32_t*>(smem_base() + kProgOff);
        const uint32_t* ps = reinterpret_cast<const uint32_t*>(&L.prog);
        for (int i = threadIdx.x; i < int(sizeof(Program) / 4); i += kThreads) {
            pd[i] = ps[i];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            KP& w = *reinterpret_cast<KP*>(dst);
            if (w.ext && w.ext[2]) {
                w.N = max(1, min(w.ext[0], w.Nb)), w.NS = max(1, min(w.ext[1], w.NSb));
            }
            w.A = w.NS * kSubset, w.np = cdiv(w.N, kTcKeys) * kTcKeys, w.chunks = cdiv(w.N * kSlots, kChunk);
            w.tc_qblocks = cdiv(w.N, kTcRows);
            w.tc_div_qblocks = w.tc_qblocks > 1 ? 0xFFFFFFFFu / uint32_t(w.tc_qblocks) + 1u : 0u;
            w.tc_div_s = w.S > 1 ? 0xFFFFFFFFu / uint32_t(w.S) + 1u : 0u;
        }
        __syncthreads();
    }
    if (threadIdx.x < 2 * kKinds) {
        reinterpret_cast<unsigned long long*>(smem_base() + kCtlOff + kTimingOff)[threadIdx.x] = 0;
    }
    gd_build();
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
    Run& r = *new (&run_state()) Run();
    // The interpreter: all of its state lives in r (shared memory), so nothing but addresses is
    // held in registers across the calls of the phase functions.
    const Program& prog = *reinterpret_cast<const Program*>(smem_base() + kProgOff);
    r.step = kp().mode == 0 ? 1 : 0;
    for (;;) {
        Flow f{r.pc, r.blk, r.step, r.ret, r.second};
        const Op op = flow_next(prog, kp(), f);
        r.pc = f.pc, r.blk = f.blk, r.step = f.step, r.ret = f.ret, r.second = f.second;
        if (op.fn == FN_END) {
            break;
        }
        if (threadIdx.x == 0) {
            CCK_TRACE_ONE(6, 0x80, op.fn);
        }
        run_op(L, r, op);
        if (threadIdx.x == 0) {
            CCK_TRACE_ONE(6, 0x82, op.fn);
        }
        r.pc++;
        if ((op.end_kind & 3) != END_NONE && grid_barrier(L, op.end_kind)) {
            break;
        }
    }
    if (smem_ctl()->quit && kp().out) {
        // The launch gave up (status word): what the schedule has left in its buffers is not a result.
        // The operator's output says so in every element instead of looking like coordinates.
        const KP& p = kp();
        const size_t n = size_t(p.S) * p.out_tokens * kSlots * kXyz;
        for (size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x; i < n; i += size_t(gridDim.x) * kThreads) {
            p.out[i] = __int_as_float(0x7fc00000);
        }
    }
    if (kp().timing && blockIdx.x == 0 && threadIdx.x == 0) {
        const unsigned long long* acc = reinterpret_cast<const unsigned long long*>(smem_base() + kCtlOff + kTimingOff);
        for (int i = 0; i < 2 * kKinds; i++) {
            kp().timing[i] += acc[i];
        }
    }
    gemm_fini();
}

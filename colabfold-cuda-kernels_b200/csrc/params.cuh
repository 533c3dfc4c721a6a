// The launch's parameter block: extents, input and scratch pointers, and the TMA tensor maps.
// It travels as one __grid_constant__ kernel parameter, so tensor maps live in parameter space.
#pragma once

#include <cuda.h>

#include "dims.cuh"

namespace cck {

// Tensor maps. A-side maps have a box of 64 bf16 x 128 rows; B-side (weight) maps a box of
// 64 bf16 x bn rows, bn chosen per GEMM on the host; both use the 128-byte swizzle. O_ maps are the
// bf16 outputs that epilogues store through TMA: box 32 columns x 32 rows, 64-byte swizzle.
#define CCK_TMAPS(X)                                                                              \
    X(A_SCT) X(A_SCH) X(A_SCLN0) X(A_SCBF) X(A_TX) X(A_TX2) X(A_TO) X(A_TC) X(A_ABF) X(A_AXQ) X(A_AXK)      \
    X(A_AO) X(A_AXHL) X(A_ACA) X(A_PC)                                                            \
    X(B_ST0_W1) X(B_ST1_W1) X(B_ST0_W2) X(B_ST1_W2) X(B_WM1) X(B_WM2) X(B_WSE)                     \
    X(B_WQKVG) X(B_WO) X(B_W1) X(B_W2) X(B_WTB) X(B_WAGGR) X(B_PLW)                                \
    X(B_ENC_WQG) X(B_ENC_WKV) X(B_ENC_WO) X(B_ENC_W1) X(B_ENC_W2)                                  \
    X(B_DEC_WQG) X(B_DEC_WKV) X(B_DEC_WO) X(B_DEC_W1) X(B_DEC_W2)                                  \
    X(T_QK) X(T_VT) X(T_PLG) X(T_TO)                                                                    \
    X(O_QKVG) X(O_AQG) X(O_AKV) X(O_TC) X(O_ACA) X(O_SCH) X(O_MODS)
#define CCK_ENUM(name) TM_##name,
enum TMap { CCK_TMAPS(CCK_ENUM) kNumTMaps };
#undef CCK_ENUM

struct TokenW {
    const float *sigma, *sc_base, *fourier_w, *fourier_b, *noise_ln, *noise_lno, *wn;
    const float *st_s[2], *st_o[2];
    const float *bm1, *bm2, *bq, *tmask, *se_b, *tb_b, *pcs, *plb, *plws, *scf, *tqkn;
    const bf16* plx;
};
struct AtomW {
    const float *amods, *apl, *bq, *qkn;
};
struct Geo {
    const float *wpos, *scq, *qmask, *kmask, *atom_mask, *tam, *wupd, *upd_b, *misc, *chir_w, *chir_a;
    const int *q2k, *tok2q, *q2ta, *chir_c, *chir_ptr, *chir_idx;
};
struct Bufs {
    float *pos, *xn, *out, *cen, *ntv, *sc, *se, *qa, *skip, *act, *tb, *upd, *agt, *grad, *kab;
    bf16 *sct, *scln0, *scbf, *sch, *mods, *ao, *abf, *aqg, *akv, *tx, *qkvg, *to, *tc, *plg;
    bf16 *axq, *axk, *axhl, *aca, *vt, *tx2;
};
// A token block runs without a grid barrier inside it: QKVG -> attention -> WO -> adaLN -> W1 -> W2,
// and the adaLN rows of the next block (or the final LayerNorm) follow W2 in the same way; the one
// barrier of a block stands between those rows and QKVG. A unit of a later operation waits for the
// units it reads, counted per block of 128 token rows: every worker warp adds one when its part of a
// unit has been stored (TX: every adaLN row of the transition's input adds one). The counters are
// zeroed at the start of a launch and count on through it: a unit of the e-th token block of the
// launch waits for (e + 1) times what one block adds.
enum FlowCnt { FC_QKVG, FC_TO, FC_TC, FC_ACT1, FC_ACT2, FC_TX, kFlowCnts };

// control words at the head of the workspace, zeroed before every launch
struct Control {
    unsigned int barrier; // arrivals of the grid barrier, monotonic; kBarrierPoison is set with the status
    unsigned int status;  // 0 ok; else the first failure (see Status)
    unsigned int where;   // grid barriers passed at the failure
    unsigned int pad;
};
// Set in the barrier word by whoever records a failure: every CTA sees it in the word it polls anyway,
// stops waiting for arrivals that will not come and leaves the schedule at its next barrier.
constexpr unsigned int kBarrierPoison = 1u << 30;
enum Status : unsigned int {
    ST_OK = 0,
    ST_BARRIER_TIMEOUT = 1, // a grid barrier gave up waiting
    ST_PIPE_TIMEOUT = 2,    // an mbarrier wait or a wait for another CTA's units gave up
};

struct KP {
    // N, NS, A, np, chunks are the real extents of this call (from ext on the device); Nb, NSb, npb
    // are the bucket's, which fix the strides of the inputs and of PLG / VT
    int S, N, A, NS, steps, nsteps, mode;
    int np, chunks;
    int Nb, NSb, npb;
    int cs, nb, tw1, aw1, nk, plc, plx;
    uint32_t flags;
    float t;      // mode 1: the noise level
    float ln_eps; // eps of the token adaLN and of the atom LayerNorms (IDSCALE: 0.1)
    int dbg_stop; // stop after this many phases of the schedule (0: never)
    uint32_t seed_lo, seed_hi;
    const int* ext; // device {N, NS, exact, seed_lo, seed_hi}, or null: the seed above is used
    TokenW tw;
    AtomW enc, dec;
    Geo geo;
    Bufs buf;
    Control* ctl;
    float* out;     // the operator's result [S][Nb][24][3], or null
    int out_tokens; // Nb
    int bn[kNumTMaps]; // box rows of each B-side map
    unsigned long long* timing; // per phase kind [wall ns, phases], or null
    unsigned int* flow_cnt; // completion counters of the token block's dependency chains (FlowCnt), flow_n each
    int flow;     // the token block's chains run on completion counters (the program was written that way)
    int flow_n;   // entries per counter array
    long long wait_cycles; // give-up limit of every wait of this launch (kWaitCycles unless a test shortened it)
    int barrier_extra;     // test hook: arrivals that the grid barriers expect on top of the grid's (0 in production)
    int attn_skew; // test hook: cycles by which the token attention's second pipeline starts late (0 in production)
    // set by the kernel with the real extents: blocks of 128 queries per sample, and the multipliers
    // that divide an item number by that and by S (n / d = umulhi(n, m) while n·d < 2^32; m = 0: d = 1)
    int tc_qblocks;
    uint32_t tc_div_qblocks, tc_div_s;
};

// phase kinds of the per-kind timing record (mk_run's `timing`): wall ns and count per kind
#define CCK_KINDS(X)                                                                               \
    X(PAIR) X(AUG) X(POS) X(INIT) X(A_LN) X(A_PROJ) X(A_ATTN) X(A_WO) X(A_LNT) X(A_W1) X(A_W2) X(A_TAIL) \
    X(AGG_GEMM) X(AGG_GATHER) X(T_ADALN) X(T_QKVG) X(T_ATTN) X(T_WO) X(T_GLU) X(T_W2) X(T_OUT) X(DEC_GLUE) X(D_ATTN) X(QKN)
#define CCK_ENUM(name) K_##name,
enum Kind { CCK_KINDS(CCK_ENUM) kKinds };
#undef CCK_ENUM

// the prepared GEMM descriptors of a launch (built on the device, block 0 of every stack)
enum Gd {
    GD_ST_W1_0, GD_ST_W1_1, GD_ST_W2_0, GD_ST_W2_1, GD_MODS_0, GD_MODS_1, GD_EMBED, GD_AGGR, GD_BROADCAST, GD_PAIR,
    GD_TOK_QKVG, GD_TOK_WO, GD_TOK_W1, GD_TOK_W2,
    GD_ENC_QG, GD_ENC_KV, GD_ENC_WO, GD_ENC_W1, GD_ENC_W2,
    GD_DEC_QG, GD_DEC_KV, GD_DEC_WO, GD_DEC_W1, GD_DEC_W2,
    kNumGd
};
enum AtomGemm { AG_QG, AG_KV, AG_WO, AG_W1, AG_W2 };
__host__ __device__ inline int gd_atom(int side, int which) {
    return (side ? GD_DEC_QG : GD_ENC_QG) + which;
}

// ---- the phase program: the host writes the schedule as a list of operations, the kernel
// interprets it. An operation runs one function over the grid; `end` says what follows it: nothing
// (the next operation shares the phase), a sub-phase barrier of this implementation, or a barrier
// that also counts as a phase of the reference's schedule (src/diffusion/sampler.cuh:99-230).
enum Fn : unsigned char {
    FN_GEMM,          // a0: descriptor, b
    FN_POS_INIT, FN_PAIR_PADS, FN_POS_CENTRE, FN_POS_AUGMENT, FN_POS_UPDATE, FN_POS_OUT_ONCE, FN_POS_OUTPUT,
    FN_POS_HEUN1, FN_POS_HEUN2, // the two halves of a Heun step
    FN_POS_MOMENTS, FN_POS_REALIGN, // REALIGN: moments of the alignment, then the aligned Euler step
    FN_NOISE_INIT,    // noise vector and atom_init at the call's noise level
    FN_SC_LN,         // a0: which of the two conditioning transitions
    FN_SC_PREP,
    FN_ATOM_LN_QK, FN_ATOM_ATTN, FN_ATOM_LN_T, // a0: side (0 encoder, 1 decoder), b
    FN_ATOM_TAIL_SKIP, FN_ATOM_TAIL_UPDATE, FN_AGGR_GATHER,
    FN_TOK_ADALN,     // a0: modulation slot, b
    FN_TOK_ADALN2,    // PARALLEL: the attention's and the transition's inputs from one LayerNorm, b
    FN_TOK_ATTN, FN_TOK_FINAL_LN, FN_DEC_INIT,
    FN_TOK_QKNORM,    // QKNORM: b
    FN_ATOM_QKNORM,   // QKNORM: a0: side, b
    FN_CTA_SYNC,      // the GEMM roles rejoin before the CTA restages shared memory
    FN_BLOCK_NEXT,    // next token block: jump to operation a0 while blocks remain
    FN_STEP_NEXT,     // next sampling step: jump to operation a0 while steps remain
    FN_CALL,          // the denoiser subroutine at operation a0; b = 1: at σ instead of t̂ (Heun's second call)
    FN_RET,
    FN_END,
};
enum OpEnd : unsigned char { END_NONE, END_SUB, END_PHASE };
constexpr unsigned char kLoopB = 255; // b comes from the token-block loop
struct Op {
    unsigned char fn, a0, b, end_kind; // end_kind: OpEnd in the low two bits, the phase kind above them
};
constexpr int kMaxOps = 124;
struct Program {
    Op ops[kMaxOps];
};

struct alignas(64) Launch {
    CUtensorMap tmap[kNumTMaps];
    KP kp;
    Program prog;
};

// ---- GEMM work descriptor: C[m][n] = A[m][k] · W[n][k]ᵀ then a fused epilogue
enum Epi : int {
    EPI_BF16,  // bf16(C + bias on the first bias_cols, sigmoid from sig_from on)
    EPI_F32,   // C + bias (optional relu) as f32
    EPI_SCRES, // out += C, f32
    EPI_RESID, // out = src + gate ⊙ C · rowmask, f32
    EPI_MODS,  // token adaLN modulations into MODS [block][slot][token][768]
    EPI_GLU,   // units of 64 columns [gate 32 | proj 32] -> silu(gate)·proj, bf16
    EPI_PAIR,  // token pair logits into PLG
};

// nfast: tile t is (row tile t / nt, column tile t % nt) instead of (t % mt, t / mt); sig: 1 + the
// completion counters (FlowCnt) that finished tiles are reported to; dep: 1 + the completion
// counters that a tile's rows of A wait for (0: none)
enum GdFlag { GF_NFAST = 1, GF_SIG_SHIFT = 4, GF_DEP_SHIFT = 8, GF_CNT_MASK = 15 };
struct GemmDesc {
    int map_a, map_b; // tensor maps
    int map_o;        // the output's store map, or -1: plain stores
    int glu_unit;     // GLU: W1 rows per unit, 64 = [gate 32 | proj 32] or 96 = [gate | proj | a_to_b]
    int a_row0;       // first row of A in its map
    int b_row0;       // first row of W in its map
    int b_kwrap;      // W's k coordinate wraps at this width (hi|lo split inputs), 0: none
    int m, n, k, bn;
    int tiles;        // cdiv(m, 128) · (n / bn)
    int mt;           // row tiles, cdiv(m, 128)
    unsigned int mt_magic; // ceil(2^32 / mt): t / mt = umulhi(t, mt_magic); 0: divide
    int epi;
    int ldo;
    void* out;
    const float* bias;
    int bias_cols, sig_from, relu;
    // RESID
    int gate_f32;
    const void* gate; // [period][..]: bf16 rows of ldg, or f32 rows of ldg
    long long ldg;
    const float* rowmask; // [period] or null
    int nt;               // column tiles, n / bn
    int fl;               // GdFlag bits
    int period;
    // MODS
    int slots, slot0, sig_slots;
    // PAIR: rows are (q, tile of 128 keys); np = key pitch of PLG, ldn = PC's row stride
    int np, ldn, ktiles, nreal, npreal;
    // BF16: the v columns of QKVG also go, transposed, into VT [sample][head·48 + d][np]
    bf16* vt;
    // what block b of a stack adds: rows of W, floats of bias, bytes of gate
    int b_step, bias_step;
    long long gate_step;
};

} // namespace cck

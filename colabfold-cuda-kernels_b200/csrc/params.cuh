// The launch's parameter block: extents, input and scratch pointers, and the TMA tensor maps.
// It travels as one __grid_constant__ kernel parameter, so tensor maps live in parameter space.
#pragma once

#include <cuda.h>

#include "dims.cuh"

namespace cck {

// Tensor maps. A-side maps have a box of 64 bf16 x 128 rows; B-side (weight) maps a box of
// 64 bf16 x bn rows, bn chosen per GEMM on the host. All use the 128-byte swizzle.
#define CCK_TMAPS(X)                                                                              \
    X(A_SCT) X(A_SCH) X(A_SCLN0) X(A_SCBF) X(A_TX) X(A_TO) X(A_TC) X(A_ABF) X(A_AXQ) X(A_AXK)      \
    X(A_AO) X(A_AXHL) X(A_ACA) X(A_PC)                                                            \
    X(B_ST0_W1) X(B_ST1_W1) X(B_ST0_W2) X(B_ST1_W2) X(B_WM1) X(B_WM2) X(B_WSE)                     \
    X(B_WQKVG) X(B_WO) X(B_W1) X(B_W2) X(B_WTB) X(B_WAGGR) X(B_PLW)                                \
    X(B_ENC_WQG) X(B_ENC_WKV) X(B_ENC_WO) X(B_ENC_W1) X(B_ENC_W2)                                  \
    X(B_DEC_WQG) X(B_DEC_WKV) X(B_DEC_WO) X(B_DEC_W1) X(B_DEC_W2)                                  \
    X(T_QK) X(T_VT) X(T_PLG)
#define CCK_ENUM(name) TM_##name,
enum TMap { CCK_TMAPS(CCK_ENUM) kNumTMaps };
#undef CCK_ENUM

struct TokenW {
    const float *sigma, *sc_base, *fourier_w, *fourier_b, *noise_ln, *noise_lno, *wn;
    const float *st_s[2], *st_o[2];
    const float *bm1, *bm2, *bq, *tmask, *se_b, *tb_b, *pcs, *plb, *plws;
    const bf16* plx;
};
struct AtomW {
    const float *amods, *apl, *bq;
};
struct Geo {
    const float *wpos, *scq, *qmask, *kmask, *atom_mask, *tam, *wupd, *upd_b, *misc;
    const int *q2k, *tok2q, *q2ta;
};
struct Bufs {
    float *pos, *xn, *out, *cen, *ntv, *sc, *se, *qa, *skip, *act, *tb, *upd, *agt;
    bf16 *sct, *scln0, *scbf, *sch, *mods, *ao, *abf, *aqg, *akv, *tx, *qkvg, *to, *tc, *plg;
    bf16 *axq, *axk, *axhl, *aca, *vt;
};

// control words at the head of the workspace, zeroed before every launch
struct Control {
    unsigned int barrier; // arrivals of the grid barrier, monotonic
    unsigned int status;  // 0 ok; else the first failure (see Status)
    unsigned int where;   // phase index at the failure
    unsigned int pad;
};
enum Status : unsigned int {
    ST_OK = 0,
    ST_BARRIER_TIMEOUT = 1, // a grid barrier gave up waiting
    ST_PIPE_TIMEOUT = 2,    // an mbarrier wait inside a CTA gave up
    ST_BAD_EXTENT = 3,      // ext asks for an extent other than the bucket's (not built yet)
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
    int dbg_stop; // stop after this many phases of the schedule (0: never)
    int attn_warp; // debug: token attention on the warp-MMA path instead of tcgen05
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
};

struct alignas(64) Launch {
    CUtensorMap tmap[kNumTMaps];
    KP kp;
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

struct GemmDesc {
    int map_a, map_b; // tensor maps
    int a_row0;       // first row of A in its map
    int b_row0;       // first row of W in its map (weights of block b start at b·n)
    int b_kwrap;      // W's k coordinate wraps at this width (hi|lo split inputs), 0: none
    int m, n, k, bn;
    int epi;
    void* out;
    int ldo;
    const float* bias;
    int bias_cols, sig_from, relu;
    // RESID
    const void* gate; // [period][..]: bf16 rows of ldg, or f32 rows of ldg
    int gate_f32;
    long long ldg;
    int period;
    const float* rowmask; // [period] or null
    const float* src;     // the residual input when it is not `out`
    // MODS
    int slots, slot0, sig_slots;
    // PAIR: rows are (q, tile of 128 keys); np = key pitch of PLG, ldn = PC's row stride
    int np, ldn, ktiles, nreal, npreal;
    const float *pcs, *plws, *plb, *tmask;
    const bf16* plx;
    // BF16: the v columns of QKVG also go, transposed, into VT [sample][head·48 + d][np]
    bf16* vt;
};

} // namespace cck

// Model constants, the operator's input order, flag bits and scratch-buffer names.
// The input order and flag values are the operator's contract with its callers
// (reference: src/diffusion/dims.cuh:46-74); everything else here is this implementation's own.
#pragma once

#include <cstddef>
#include <cstdint>

namespace cck {

typedef uint16_t bf16; // raw bits

constexpr int kTokC = 768, kHeads = 16, kHeadD = 48, kQKVG = 4 * kTokC, kTokHidden = 2 * kTokC;
constexpr int kTokModSlots = 6, kTokMods1 = 4;
constexpr int kAtomC = 128, kAtomHeads = 4, kAtomHeadD = 32, kAtomHidden = 2 * kAtomC;
constexpr int kSubset = 32, kSubsetKeys = 128, kAtomModSlots = 8, kAtomBlocks = 3;
constexpr int kSlots = 24, kFourier = 256, kGluHalf = 32, kXyz = 3;
constexpr int kNbMax = 24, kPairHeads = kHeads;
constexpr int kChunk = 1024; // position slots per deterministic reduction chunk
constexpr int kCenSums = 4;
constexpr float kSigmaData = 16.0f, kMaskBias = 1e9f, kLnEps = 1e-5f;
constexpr float kLog2e = 1.4426950408889634f;

constexpr int kThreads = 384; // 12 warps: TMA, MMA and 8 workers in the tensor-core phases, a second TMA and MMA in the token attention; all of them in row phases
constexpr int kWarps = kThreads / 32;

// flag bits of the `flags` attribute (reference: src/diffusion/dims.cuh:46-57)
enum Flag : uint32_t {
    F_CHAIN_K = 1, F_ATOB = 2, F_QKNORM = 4, F_PARALLEL = 8, F_CHIRAL = 16, F_IDSCALE = 32,
    F_SCFINAL = 64, F_HEUN = 128, F_ESM = 256, F_REALIGN = 512,
};
// Bits 0-9 are the reference's. Bits 16-23 are set aside for variants that only this library has (none
// is built: weights held in FP8-e4m3 would be bit 16); a bit outside both ranges is refused as unknown.
constexpr uint32_t kReferenceFlagBits = 0x3FFu, kExtensionFlagBits = 0xFF0000u;
constexpr uint32_t kSupportedFlags = F_HEUN | F_SCFINAL | F_IDSCALE | F_CHAIN_K | F_QKNORM | F_PARALLEL | F_ATOB | F_REALIGN | F_CHIRAL;
constexpr float kChiralEps = 1e-6f; // CHIRAL: eps of the dihedral's construction (reference: src/diffusion/positions.cuh:15)
// REALIGN: partial moments per chunk (w, w·x, w·den, w·x·denᵀ) and the Jacobi iteration's bounds
// (reference: src/diffusion/dims.cuh:40, src/diffusion/positions.cuh:16-17)
constexpr int kMoments = 16, kJacobiSweeps = 16;
constexpr float kTiny = 1e-30f;
// rows of a QKNORM table (reference: src/diffusion/dims.cuh:112)
enum QkNorm { QKN_Q_SCALE, QKN_Q_OFFSET, QKN_K_SCALE, QKN_K_OFFSET, kQkNormRows }; // the other variant bits are rejected until they are built
constexpr float kIdScaleEps = 0.1f; // IDSCALE: eps of the token adaLN and of the atom LayerNorms (reference: src/diffusion/dims.cuh:43)
// HEUN: the churn window on the previous noise level and the floor under the added noise's variance
// (reference: src/diffusion/positions.cuh:11-13)
constexpr float kChurnMin = 4e-4f, kChurnMax = 80.f, kHeunFloor = 1e-6f;

// the 74 inputs in call order (reference: src/diffusion/dims.cuh:61-74)
#define CCK_INPUTS(X)                                                                             \
    X(SIGMA) X(SC_BASE) X(FOURIER_W) X(FOURIER_B) X(NOISE_LN) X(WN)                               \
    X(ST0_S) X(ST0_O) X(ST0_W1) X(ST0_W2) X(ST1_S) X(ST1_O) X(ST1_W1) X(ST1_W2)                   \
    X(WM1) X(BM1) X(WM2) X(BM2) X(WSE)                                                            \
    X(WQKVG) X(BQ) X(WO) X(W1) X(W2) X(PC) X(TMASK) X(WTB)                                        \
    X(WPOS) X(SCQ) X(QMASK) X(KMASK) X(Q2K) X(TOK2Q) X(Q2TA) X(ATOM_MASK) X(TAM) X(WAGGR) X(WUPD) \
    X(ENC_AMODS) X(ENC_APL) X(ENC_WQG) X(ENC_BQ) X(ENC_WKV) X(ENC_WO) X(ENC_W1) X(ENC_W2)         \
    X(DEC_AMODS) X(DEC_APL) X(DEC_WQG) X(DEC_BQ) X(DEC_WKV) X(DEC_WO) X(DEC_W1) X(DEC_W2)         \
    X(NOISE_LNO) X(SE_B) X(TB_B) X(UPD_B) X(SCF) X(ROPE)                                          \
    X(PCS) X(PLW) X(PLB) X(PLWS) X(PLX)                                                           \
    X(TQKN) X(EQKN) X(DQKN) X(CHIR_W) X(CHIR_C) X(CHIR_A) X(CHIR_PTR) X(CHIR_IDX)                 \
    X(MISC)
#define CCK_ENUM(name) IN_##name,
enum In { CCK_INPUTS(CCK_ENUM) kNumInputs };
#undef CCK_ENUM
static_assert(kNumInputs == 74, "the operator takes 74 inputs after ext");
constexpr int kAtomInputs = IN_DEC_AMODS - IN_ENC_AMODS; // AMODS, APL, WQG, BQ, WKV, WO, W1, W2

enum Misc { M_GAMMA0, M_GAMMA_MIN, M_NOISE_SCALE, M_STEP_SCALE, M_FLAGS, M_CHURN };
enum TokMod { TM_ATTN_SCALE, TM_ATTN_BIAS, TM_TRANS_SCALE, TM_TRANS_BIAS, TM_ATTN_GATE, TM_TRANS_GATE };
enum AtomMod { AM_Q_SCALE, AM_Q_BIAS, AM_K_SCALE, AM_K_BIAS, AM_T_SCALE, AM_T_BIAS, AM_ATTN_GATE, AM_T_GATE };

// Scratch buffers in workspace order. The first 29 keep the reference's names and meaning
// (reference: src/diffusion/dims.cuh:80-86) so that the same debug reads work on either library;
// PLG has this implementation's own layout ([table][head][np][np] bf16, row-major). The rest are
// this implementation's staging buffers.
#define CCK_BUFFERS(X)                                                                            \
    X(POS) X(XN) X(OUT) X(GRAD) X(CEN) X(KAB) X(NTV) X(SC) X(SCT) X(SCLN0) X(SCBF) X(SCH) X(MODS)  \
    X(SE) X(QA) X(SKIP) X(AO) X(ABF) X(AQG) X(AKV) X(ACT) X(TX) X(TX2) X(QKVG) X(TO) X(TC) X(TB)  \
    X(UPD) X(PLG) X(AXQ) X(AXK) X(AXHL) X(ACA) X(AGT) X(VT) X(FLOW)
#define CCK_ENUM(name) B_##name,
enum Buf { CCK_BUFFERS(CCK_ENUM) kNumBufs };
#undef CCK_ENUM

} // namespace cck

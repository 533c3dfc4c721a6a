// Host side: shape checks, the workspace layout, TMA tensor maps, the launch, the plain C entry
// points and the ctypes debug API. The product path has no CPU fallback: every entry point either
// enqueues the sm_100a kernel or returns an error.
//
// The interfaces mirror the reference's host glue (src/diffusion/host.cuh:19-499): widths are
// derived from the inputs' byte sizes, the caller owns every buffer, nothing is allocated or
// synchronised on the operator path.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "sampler.cuh"

namespace cck {

constexpr size_t kAlign = 256;
constexpr int kMaxDevices = 64;

inline size_t align_up(size_t x, size_t a) {
    return (x + a - 1) / a * a;
}
inline int pad_keys(int n) {
    return cdiv(n, kTcKeys) * kTcKeys;
}

static const char* const kBufNames[] = {
#define CCK_NAME(name) #name,
    CCK_BUFFERS(CCK_NAME)
#undef CCK_NAME
};

// error codes of the C entry points
enum Err : int {
    E_OK = 0,
    E_ARITY = 1,     // wrong number of inputs
    E_WORKSPACE = 2, // workspace too small
    E_SHAPE = 3,     // byte sizes that do not fit one model
    E_FLAGS = 4,     // a variant flag that is not built
    E_LAUNCH = 5,    // CUDA error at launch
    E_DEVICE = 6,    // not an sm_100 device, or the driver lacks tensor-map encoding
    E_STATE = 7,     // debug API used before mk_setup
    E_KERNEL = 8,    // the kernel reported a failure in its status word
};
static thread_local std::string g_error;
inline int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

// Everything that depends only on the shapes: model widths and the workspace layout
struct Template {
    int S, Nb, NSb, nsteps;
    uint32_t flags;
    int steps, cs, nb, tw1, aw1, nk, plc, plx, np, flow_n;
    size_t off[kNumBufs], bytes[kNumBufs];
    size_t total;
};

// widths from byte sizes (reference: src/diffusion/host.cuh:74-89), then every size is checked
static int make_template(Template& t, int S, int Nb, int NSb, int nsteps, uint32_t flags, const size_t* in) {
    t = Template{};
    t.S = S, t.Nb = Nb, t.NSb = NSb, t.nsteps = nsteps, t.flags = flags;
    if (flags & ~(kReferenceFlagBits | kExtensionFlagBits)) {
        return fail(E_FLAGS, "MkSample: flags " + std::to_string(flags) + " set bits that no variant uses");
    }
    if (flags & ~kSupportedFlags) {
        return fail(E_FLAGS, "MkSample: flags " + std::to_string(flags) + " ask for a variant that is not built");
    }
    if (S < 1 || Nb < 1 || NSb < 1 || nsteps < 0) {
        return fail(E_SHAPE, "MkSample: samples, tokens and subsets must be positive");
    }
    t.steps = int(in[IN_SIGMA] / sizeof(float)) - 1;
    t.cs = int(in[IN_SC_BASE] / (size_t(Nb) * sizeof(float)));
    t.nb = int(in[IN_WQKVG] / (size_t(kQKVG) * kTokC * sizeof(bf16)));
    t.tw1 = t.nb ? int(in[IN_W1] / (size_t(t.nb) * kTokC * sizeof(bf16))) : 0;
    t.aw1 = int(in[IN_ENC_W1] / (size_t(kAtomBlocks) * kAtomC * sizeof(bf16)));
    t.nk = int(in[IN_Q2K] / (size_t(NSb) * sizeof(int)));
    t.plc = t.nb ? int(in[IN_PLW] / (size_t(t.nb) * kPairHeads * sizeof(bf16))) : 0;
    t.plx = in[IN_PLX] == size_t(Nb) * Nb * sizeof(bf16);
    t.np = pad_keys(Nb);
    if (t.cs != 384 || t.nb < 1 || t.nb > kNbMax || (t.tw1 != 2 * kTokHidden && t.tw1 != 3 * kTokHidden) || t.aw1 != (flags & F_ATOB ? 3 : 2) * kAtomHidden ||
        t.nk != kSubsetKeys || t.plc < kBK || t.plc % kBK || nsteps > t.steps) {
        return fail(E_SHAPE, "MkSample: widths derived from the inputs' sizes are not a supported model");
    }
    if ((flags & F_QKNORM) && (in[IN_TQKN] != size_t(t.nb) * kQkNormRows * kTokC * sizeof(float) ||
                               in[IN_EQKN] != size_t(kAtomBlocks) * kQkNormRows * kAtomC * sizeof(float) || in[IN_DQKN] != in[IN_EQKN])) {
        return fail(E_SHAPE, "MkSample: inputs 65-67 (TQKN, EQKN, DQKN) have the wrong size for the QKNORM variant");
    }
    if ((flags & F_CHIRAL) && (in[IN_CHIR_W] != size_t(kXyz) * kAtomC * sizeof(float) || in[IN_CHIR_PTR] != (size_t(Nb) * kSlots + 1) * sizeof(int) ||
                               in[IN_CHIR_C] != 4 * in[IN_CHIR_A] || in[IN_CHIR_A] < sizeof(float) || in[IN_CHIR_IDX] < sizeof(int))) {
        return fail(E_SHAPE, "MkSample: inputs 68-72 (CHIR_*) have the wrong sizes for the CHIRAL variant");
    }
    if ((flags & F_SCFINAL) && in[IN_SCF] != 2 * size_t(t.cs) * sizeof(float)) {
        return fail(E_SHAPE, "MkSample: input 58 (SCF) has the wrong size for the SCFINAL variant");
    }
    const size_t A = size_t(NSb) * kSubset, nb = t.nb, cs = t.cs, f = sizeof(float), h = sizeof(bf16), i4 = sizeof(int);
    struct {
        int id;
        size_t want;
    } sizes[] = {
        {IN_SC_BASE, Nb * cs * f}, {IN_FOURIER_W, kFourier * f}, {IN_FOURIER_B, kFourier * f},
        {IN_NOISE_LN, kFourier * f}, {IN_NOISE_LNO, kFourier * f}, {IN_WN, kFourier * cs * f},
        {IN_ST0_S, cs * f}, {IN_ST0_O, cs * f}, {IN_ST0_W1, 4 * cs * cs * h}, {IN_ST0_W2, 2 * cs * cs * h},
        {IN_ST1_S, cs * f}, {IN_ST1_O, cs * f}, {IN_ST1_W1, 4 * cs * cs * h}, {IN_ST1_W2, 2 * cs * cs * h},
        {IN_WM1, nb * kTokMods1 * kTokC * cs * h}, {IN_BM1, nb * kTokMods1 * kTokC * f},
        {IN_WM2, nb * 2 * kTokC * cs * h}, {IN_BM2, nb * 2 * kTokC * f}, {IN_WSE, kTokC * cs * h}, {IN_SE_B, kTokC * f},
        {IN_WQKVG, nb * kQKVG * kTokC * h}, {IN_BQ, nb * kTokC * f}, {IN_WO, nb * kTokC * kTokC * h},
        {IN_W1, nb * size_t(t.tw1) * kTokC * h}, {IN_W2, nb * kTokC * kTokHidden * h},
        {IN_PC, size_t(Nb) * Nb * t.plc * h}, {IN_PCS, size_t(Nb) * Nb * 2 * f}, {IN_TMASK, Nb * f},
        {IN_PLW, nb * kPairHeads * t.plc * h}, {IN_PLB, nb * kPairHeads * f}, {IN_PLWS, nb * kPairHeads * f},
        {IN_WTB, kAtomC * kTokC * h}, {IN_TB_B, kAtomC * f}, {IN_WPOS, kXyz * kAtomC * f}, {IN_SCQ, A * kAtomC * f},
        {IN_QMASK, A * f}, {IN_KMASK, size_t(NSb) * t.nk * f}, {IN_Q2K, size_t(NSb) * t.nk * i4}, {IN_TOK2Q, A * i4},
        {IN_Q2TA, size_t(Nb) * kSlots * i4}, {IN_ATOM_MASK, size_t(Nb) * kSlots * f}, {IN_TAM, size_t(Nb) * kSlots * f},
        {IN_WAGGR, kTokC * kAtomC * h}, {IN_WUPD, kXyz * kAtomC * f}, {IN_UPD_B, kXyz * f}, {IN_MISC, 6 * f},
    };
    for (const auto& s : sizes) {
        if (in[s.id] != s.want) {
            return fail(E_SHAPE, std::string("MkSample: input ") + std::to_string(s.id) + " has " +
                                     std::to_string(in[s.id]) + " bytes, expected " + std::to_string(s.want));
        }
    }
    for (int side = 0; side < 2; side++) {
        const int i0 = side ? IN_DEC_AMODS : IN_ENC_AMODS;
        const size_t want[kAtomInputs] = {
            kAtomBlocks * A * kAtomModSlots * kAtomC * f,
            kAtomBlocks * size_t(NSb) * kAtomHeads * kSubset * t.nk * f,
            kAtomBlocks * 2 * kAtomC * kAtomC * h,
            kAtomBlocks * kAtomC * f,
            kAtomBlocks * 2 * kAtomC * kAtomC * h,
            kAtomBlocks * kAtomC * kAtomC * h,
            kAtomBlocks * size_t(t.aw1) * kAtomC * h,
            kAtomBlocks * kAtomC * kAtomHidden * h,
        };
        for (int j = 0; j < kAtomInputs; j++) {
            if (in[i0 + j] != want[j]) {
                return fail(E_SHAPE, std::string("MkSample: atom input ") + std::to_string(i0 + j) + " has " +
                                         std::to_string(in[i0 + j]) + " bytes, expected " + std::to_string(want[j]));
            }
        }
    }

    const size_t rt = size_t(S) * Nb, ra = size_t(S) * A, pos = size_t(S) * Nb * kSlots;
    const size_t chunks = size_t(S) * cdiv(Nb * kSlots, kChunk);
    size_t want[kNumBufs] = {};
    want[B_POS] = want[B_XN] = want[B_OUT] = pos * kXyz * f;
    want[B_GRAD] = flags & (F_HEUN | F_REALIGN) ? pos * kXyz * f : 0; // Heun's first slope, or REALIGN's denoised positions
    want[B_KAB] = flags & F_REALIGN ? chunks * kMoments * f : 0;
    want[B_CEN] = chunks * kCenSums * f;
    want[B_NTV] = cs * f;
    want[B_SC] = Nb * cs * f;
    want[B_SCT] = want[B_SCLN0] = want[B_SCBF] = Nb * cs * h;
    want[B_SCH] = Nb * 2 * cs * h;
    want[B_MODS] = nb * kTokModSlots * Nb * kTokC * h;
    want[B_SE] = size_t(Nb) * kTokC * f;
    want[B_QA] = want[B_SKIP] = ra * kAtomC * f;
    want[B_AO] = want[B_ABF] = want[B_AXQ] = want[B_AXK] = ra * kAtomC * h;
    want[B_AQG] = want[B_AKV] = want[B_AXHL] = want[B_ACA] = ra * 2 * kAtomC * h;
    want[B_ACT] = rt * kTokC * f;
    want[B_TX] = want[B_TO] = rt * kTokC * h;
    want[B_TX2] = flags & F_PARALLEL ? rt * kTokC * h : 0; // the transition's input beside the attention's
    want[B_QKVG] = rt * kQKVG * h;
    want[B_TC] = rt * kTokHidden * h;
    want[B_TB] = rt * kAtomC * f;
    want[B_UPD] = ra * kXyz * f;
    want[B_PLG] = nb * kPairHeads * size_t(t.np) * t.np * h;
    want[B_AGT] = ra * kTokC * f;
    want[B_VT] = size_t(S) * kTokC * t.np * h;
    t.flow_n = int(cdiv(int(rt), kBM)) + 1;
    want[B_FLOW] = size_t(kFlowCnts) * t.flow_n * sizeof(unsigned int);
    size_t off = align_up(sizeof(Control), kAlign);
    for (int b = 0; b < kNumBufs; b++) {
        t.off[b] = off, t.bytes[b] = want[b];
        off = align_up(off + want[b], kAlign);
    }
    t.total = off;
    return E_OK;
}

// ---- per-device state: SM count, kernel attributes, the tensor-map encoder
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct Device {
    bool ready = false;
    int sms = 0;
};
static std::mutex g_mutex;
static bool g_flow = true; // mk_set_flow: the token block's chains on completion counters (default) or on barriers
static long long g_wait_cycles = 0; // mk_set_wait_test: a test's give-up limit (0: the default)
static int g_barrier_extra = 0;     // mk_set_wait_test: arrivals that no CTA will make, so that the first grid barrier runs out
static int g_attn_skew = 0; // mk_set_attn_skew: a test's delay (cycles) of the token attention's second pipeline
static Device g_device[kMaxDevices];
static EncodeTiled g_encode = nullptr;

static int device_state(Device& out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return fail(E_DEVICE, "MkSample: no CUDA device");
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    Device& d = g_device[dev];
    if (!d.ready) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess || prop.major != 10) {
            return fail(E_DEVICE, "MkSample: this library holds sm_100a code only");
        }
        d.sms = prop.multiProcessorCount;
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
                return fail(E_DEVICE, "MkSample: the driver has no cuTensorMapEncodeTiled");
            }
            g_encode = reinterpret_cast<EncodeTiled>(fn);
        }
        if (cudaFuncSetAttribute(reinterpret_cast<const void*>(cck_sampler_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc) != cudaSuccess) {
            return fail(E_DEVICE, "MkSample: cannot reserve shared memory for the sampler kernel");
        }
        d.ready = true;
    }
    out = d;
    return E_OK;
}

// a [rows][cols] bf16 matrix with row pitch ld (elements), box = 64 columns x box_rows, 128-byte swizzle
static int encode_map(CUtensorMap* m, const void* base, size_t rows, size_t cols, size_t ld, int box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * sizeof(bf16)};
    const cuuint32_t box[2] = {kBK, cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(E_LAUNCH, "MkSample: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
    }
    return E_OK;
}

// a bf16 output [rows][cols] stored by epilogues in blocks of 32 rows x 32 columns (64-byte rows in
// shared memory, 64-byte swizzle)
static int encode_store_map(CUtensorMap* m, const void* base, size_t rows, size_t cols) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * sizeof(bf16)};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(E_LAUNCH, "MkSample: cuTensorMapEncodeTiled failed for a store map (" + std::to_string(int(r)) + ")");
    }
    return E_OK;
}

// a bf16 output [rows][cols] stored in boxes of box_rows x box_cols from dense rows in shared memory
static int encode_rows_store_map(CUtensorMap* m, const void* base, size_t rows, size_t cols, int box_rows, int box_cols) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * sizeof(bf16)};
    const cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(E_LAUNCH, "MkSample: cuTensorMapEncodeTiled failed for a row store map (" + std::to_string(int(r)) + ")");
    }
    return E_OK;
}

// the column tile of a GEMM: the widest of 256/128/64 that divides n, unless a narrower one needs
// fewer whole rounds over the grid (weighted by width)
// (GLU GEMMs whose units have 96 rows take 192 or 96)
inline int choose_bn(size_t m, int n, int grid, int max_bn = kMaxBN, int unit = 64) {
    int best = unit;
    double best_cost = 1e300;
    for (int bn = 4 * unit; bn >= unit; bn /= 2) {
        if (n % bn || bn > max_bn) {
            continue;
        }
        const size_t tiles = (m + kBM - 1) / kBM * size_t(n / bn);
        const double cost = double((tiles + grid - 1) / grid) * (bn + 24);
        if (cost < best_cost) {
            best_cost = cost, best = bn;
        }
    }
    return best;
}

// ---- the phase program (the schedule of the reference, src/diffusion/sampler.cuh:87-230, flags = 0,
// with this implementation's sub-phases)
struct ProgramWriter {
    Program& pr;
    int n = 0;
    explicit ProgramWriter(Program& p) : pr(p) {}
    // the operation; `end` and `kind` say which barrier follows it
    void op(int fn, int a0 = 0, int b = 0, int end = END_NONE, int kind = 0) {
        if (n < kMaxOps) {
            Op& o = pr.ops[n];
            o.fn = (unsigned char)fn, o.a0 = (unsigned char)a0, o.b = (unsigned char)b, o.end_kind = (unsigned char)(end | kind << 2);
        }
        n++;
    }
    void gemm(int id, int b = 0, int end = END_NONE, int kind = 0) {
        op(FN_GEMM, id, b, end, kind);
    }
};
// one denoiser call (reference: src/diffusion/sampler.cuh:137-182)
// kProgFlow (a bit of `flags` that only the program writer knows): a token block runs as one phase, its
// operations chained by completion counters (FlowCnt) instead of barriers. Not with PARALLEL or QKNORM, whose blocks have other phases; not in a debug run that
// stops at a phase of the reference's schedule, which counts the barriers.
constexpr uint32_t kProgFlow = 1u << 30;
inline bool flow_allowed(uint32_t flags) {
    return !(flags & (F_PARALLEL | F_QKNORM));
}
static void write_denoise(ProgramWriter& w, uint32_t flags) {
    const bool qkn = flags & F_QKNORM, par = flags & F_PARALLEL;
    const bool flow = (flags & kProgFlow) && flow_allowed(flags);
    // conditioning + atom encoder + aggregation
    w.op(FN_NOISE_INIT, 0, 0, END_PHASE, K_INIT);
    for (int b = 0; b < kAtomBlocks; b++) {
        if (b < 2) {
            w.op(FN_SC_LN, b);
        } else {
            w.op(FN_SC_PREP);
        }
        if (par) { // the transition's input comes from the block input too: both adaLN passes first
            w.op(FN_ATOM_LN_QK, 0, b);
            w.op(FN_ATOM_LN_T, 0, b, END_SUB, K_A_LN);
        } else {
            w.op(FN_ATOM_LN_QK, 0, b, END_SUB, K_A_LN);
        }
        w.gemm(gd_atom(0, AG_QG), b);
        if (qkn) { // LayerNorm of the q and k just written, before the phase ends
            w.gemm(gd_atom(0, AG_KV), b, END_SUB, K_A_PROJ);
            w.op(FN_ATOM_QKNORM, 0, b, END_PHASE, K_QKN);
        } else {
            w.gemm(gd_atom(0, AG_KV), b, END_PHASE, K_A_PROJ);
        }
        // the conditioning's GEMMs ride in the attention phase
        if (b < 2) {
            w.gemm(GD_ST_W1_0 + b);
        } else {
            w.gemm(GD_MODS_0), w.gemm(GD_MODS_1), w.gemm(GD_EMBED);
        }
        w.op(FN_CTA_SYNC);
        w.op(FN_ATOM_ATTN, 0, b, END_PHASE, K_A_ATTN);
        if (b < 2) {
            w.gemm(GD_ST_W2_0 + b);
        }
        w.gemm(gd_atom(0, AG_WO), b, END_SUB, K_A_WO);
        if (!par) {
            w.op(FN_ATOM_LN_T, 0, b, END_SUB, K_A_LNT);
        }
        w.gemm(gd_atom(0, AG_W1), b, END_SUB, K_A_W1);
        if (b + 1 < kAtomBlocks) {
            w.gemm(gd_atom(0, AG_W2), b, END_PHASE, K_A_W2);
        } else {
            w.gemm(gd_atom(0, AG_W2), b, END_SUB, K_A_W2);
            w.op(FN_ATOM_TAIL_SKIP, 0, 0, END_PHASE, K_A_TAIL);
        }
    }
    w.gemm(GD_AGGR, 0, END_SUB, K_AGG_GEMM);
    w.op(FN_AGGR_GATHER, 0, 0, END_PHASE, K_AGG_GATHER);
    // the token blocks (reference: src/diffusion/sampler.cuh:99-134)
    const int block0 = w.n;
    if (par) { // reference: src/diffusion/sampler.cuh:101-127: both residual branches read the block input
        w.op(FN_TOK_ADALN2, 0, kLoopB, END_PHASE, K_T_ADALN);
        w.gemm(GD_TOK_QKVG, kLoopB);
        w.gemm(GD_TOK_W1, kLoopB, END_PHASE, K_T_QKVG);
        if (qkn) {
            w.op(FN_TOK_QKNORM, 0, kLoopB, END_PHASE, K_QKN);
        }
        w.gemm(GD_TOK_W2, kLoopB);
        w.op(FN_CTA_SYNC);
        w.op(FN_TOK_ATTN, 0, kLoopB, END_PHASE, K_T_ATTN);
        w.gemm(GD_TOK_WO, kLoopB, END_PHASE, K_T_WO);
    } else if (flow) {
        w.op(FN_TOK_ADALN, TM_ATTN_SCALE, kLoopB, END_PHASE, K_T_W2);
        w.gemm(GD_TOK_QKVG, kLoopB);
        w.op(FN_CTA_SYNC);
        w.op(FN_TOK_ATTN, 0, kLoopB);
        w.op(FN_CTA_SYNC);
        w.gemm(GD_TOK_WO, kLoopB);
        w.op(FN_TOK_ADALN, TM_TRANS_SCALE, kLoopB); // its rows wait for WO's tiles over them
        // (WO's epilogue keeps the residual rows it fetched ahead in the upper halves of the ring's
        // weight slots, which W1's 256-column tiles fill: every warp of the CTA is through with WO first)
        w.op(FN_CTA_SYNC);
        w.gemm(GD_TOK_W1, kLoopB); // a tile waits for the adaLN rows of its block of 128
        w.gemm(GD_TOK_W2, kLoopB); // the next block's adaLN rows (or the final LayerNorm's) wait for its tiles
    } else {
        w.op(FN_TOK_ADALN, TM_ATTN_SCALE, kLoopB, END_PHASE, K_T_ADALN);
        w.gemm(GD_TOK_QKVG, kLoopB, END_PHASE, K_T_QKVG);
        if (qkn) { // a phase of its own in the reference's schedule too (src/diffusion/sampler.cuh:114-117)
            w.op(FN_TOK_QKNORM, 0, kLoopB, END_PHASE, K_QKN);
        }
        w.op(FN_TOK_ATTN, 0, kLoopB, END_PHASE, K_T_ATTN);
        w.gemm(GD_TOK_WO, kLoopB, END_PHASE, K_T_WO);
        w.op(FN_TOK_ADALN, TM_TRANS_SCALE, kLoopB, END_PHASE, K_T_ADALN);
        w.gemm(GD_TOK_W1, kLoopB, END_PHASE, K_T_GLU);
        w.gemm(GD_TOK_W2, kLoopB, END_PHASE, K_T_W2);
    }
    w.op(FN_BLOCK_NEXT, block0);
    // back to atoms + atom decoder
    w.op(FN_TOK_FINAL_LN, 0, 0, END_PHASE, K_T_OUT);
    w.gemm(GD_BROADCAST, 0, END_PHASE, K_T_OUT);
    w.op(FN_DEC_INIT, 0, 0, END_PHASE, K_DEC_GLUE);
    for (int b = 0; b < kAtomBlocks; b++) {
        if (par) { // the transition's input comes from the block input too: both adaLN passes first
            w.op(FN_ATOM_LN_QK, 1, b);
            w.op(FN_ATOM_LN_T, 1, b, END_SUB, K_A_LN);
        } else {
            w.op(FN_ATOM_LN_QK, 1, b, END_SUB, K_A_LN);
        }
        w.gemm(gd_atom(1, AG_QG), b);
        if (qkn) {
            w.gemm(gd_atom(1, AG_KV), b, END_SUB, K_A_PROJ);
            w.op(FN_ATOM_QKNORM, 1, b, END_PHASE, K_QKN);
        } else {
            w.gemm(gd_atom(1, AG_KV), b, END_PHASE, K_A_PROJ);
        }
        w.op(FN_ATOM_ATTN, 1, b, END_PHASE, K_D_ATTN);
        w.gemm(gd_atom(1, AG_WO), b, END_SUB, K_A_WO);
        if (!par) {
            w.op(FN_ATOM_LN_T, 1, b, END_SUB, K_A_LNT);
        }
        w.gemm(gd_atom(1, AG_W1), b, END_SUB, K_A_W1);
        if (b + 1 < kAtomBlocks) {
            w.gemm(gd_atom(1, AG_W2), b, END_PHASE, K_A_W2);
        } else {
            w.gemm(gd_atom(1, AG_W2), b, END_SUB, K_A_W2);
            w.op(FN_ATOM_TAIL_UPDATE, 0, 0, END_PHASE, K_A_TAIL);
        }
    }
}
// mode 0: the sampling loop (reference: src/diffusion/sampler.cuh:184-217, Euler path);
// mode 1: one denoiser call on the caller's XN at t, denoised positions to OUT (:219-230)
static int make_program(Program& pr, int mode, int nsteps, uint32_t flags) {
    memset(&pr, 0, sizeof pr);
    ProgramWriter w(pr);
    int calls[3], ncalls = 0; // the CALL operations, patched with the subroutine's address below
    if (mode == 0) {
        w.op(FN_POS_INIT);
    }
    w.op(FN_PAIR_PADS);
    w.gemm(GD_PAIR, 0, END_PHASE, K_PAIR);
    if (mode == 0 && nsteps > 0) {
        const int step0 = w.n;
        w.op(FN_POS_CENTRE, 0, 0, END_PHASE, K_AUG);
        w.op(FN_POS_AUGMENT, 0, 0, END_PHASE, K_AUG);
        calls[ncalls++] = w.n;
        w.op(FN_CALL, 0, 0);
        if (flags & F_REALIGN) { // reference: src/diffusion/sampler.cuh:200-203 (it takes precedence over HEUN there too)
            w.op(FN_POS_MOMENTS, 0, 0, END_PHASE, K_POS);
            w.op(FN_POS_REALIGN, 0, 0, END_PHASE, K_POS);
        } else if (flags & F_HEUN) { // two denoiser calls per step (reference: src/diffusion/sampler.cuh:204-209)
            w.op(FN_POS_HEUN1, 0, 0, END_PHASE, K_POS);
            calls[ncalls++] = w.n;
            w.op(FN_CALL, 0, 1);
            w.op(FN_POS_HEUN2, 0, 0, END_PHASE, K_POS);
        } else {
            w.op(FN_POS_UPDATE, 0, 0, END_PHASE, K_POS);
        }
        w.op(FN_STEP_NEXT, step0);
    }
    if (mode == 0) {
        w.op(FN_POS_OUTPUT);
    } else {
        calls[ncalls++] = w.n;
        w.op(FN_CALL, 0, 0);
        w.op(FN_POS_OUT_ONCE, 0, 0, END_PHASE, K_POS);
    }
    w.op(FN_END);
    const int sub = w.n;
    write_denoise(w, flags);
    w.op(FN_RET);
    if (w.n > kMaxOps || sub > 255) {
        return fail(E_LAUNCH, "MkSample: the phase program outgrew its table");
    }
    for (int i = 0; i < ncalls; i++) {
        pr.ops[calls[i]].a0 = (unsigned char)sub;
    }
    return E_OK;
}

// the launch block for one call
static int make_launch(Launch& L, const Template& t, const Device& dev, const void* const* in, char* ws, float* out,
                       const int* ext) {
    memset(&L, 0, sizeof L);
    KP& p = L.kp;
    const int N = t.Nb, A = t.NSb * kSubset;
    p.S = t.S, p.N = N, p.NS = t.NSb, p.A = A, p.steps = t.steps, p.nsteps = t.nsteps;
    p.np = t.np, p.chunks = cdiv(N * kSlots, kChunk);
    p.Nb = t.Nb, p.NSb = t.NSb, p.npb = t.np;
    p.cs = t.cs, p.nb = t.nb, p.tw1 = t.tw1, p.aw1 = t.aw1, p.nk = t.nk, p.plc = t.plc, p.plx = t.plx;
    p.ln_eps = t.flags & F_IDSCALE ? kIdScaleEps : kLnEps;
    p.flags = t.flags, p.ext = ext, p.out = out, p.out_tokens = t.Nb;
    p.flow = g_flow && flow_allowed(t.flags), p.flow_n = t.flow_n;
    p.attn_skew = g_attn_skew, p.wait_cycles = g_wait_cycles > 0 ? g_wait_cycles : kWaitCycles, p.barrier_extra = g_barrier_extra;
    auto F = [&](int i) { return static_cast<const float*>(in[i]); };
    auto H = [&](int i) { return static_cast<const bf16*>(in[i]); };
    auto I = [&](int i) { return static_cast<const int*>(in[i]); };
    TokenW& w = p.tw;
    w.sigma = F(IN_SIGMA), w.sc_base = F(IN_SC_BASE), w.fourier_w = F(IN_FOURIER_W), w.fourier_b = F(IN_FOURIER_B);
    w.noise_ln = F(IN_NOISE_LN), w.noise_lno = F(IN_NOISE_LNO), w.wn = F(IN_WN);
    w.st_s[0] = F(IN_ST0_S), w.st_o[0] = F(IN_ST0_O), w.st_s[1] = F(IN_ST1_S), w.st_o[1] = F(IN_ST1_O);
    w.bm1 = F(IN_BM1), w.bm2 = F(IN_BM2), w.bq = F(IN_BQ), w.tmask = F(IN_TMASK), w.se_b = F(IN_SE_B), w.scf = F(IN_SCF), w.tqkn = F(IN_TQKN);
    w.tb_b = F(IN_TB_B), w.pcs = F(IN_PCS), w.plb = F(IN_PLB), w.plws = F(IN_PLWS), w.plx = H(IN_PLX);
    for (int side = 0; side < 2; side++) {
        AtomW& a = side ? p.dec : p.enc;
        const int i0 = side ? IN_DEC_AMODS : IN_ENC_AMODS;
        a.amods = F(i0), a.apl = F(i0 + 1), a.bq = F(i0 + 3), a.qkn = F(side ? IN_DQKN : IN_EQKN);
    }
    Geo& g = p.geo;
    g.wpos = F(IN_WPOS), g.scq = F(IN_SCQ), g.qmask = F(IN_QMASK), g.kmask = F(IN_KMASK);
    g.atom_mask = F(IN_ATOM_MASK), g.tam = F(IN_TAM), g.wupd = F(IN_WUPD), g.upd_b = F(IN_UPD_B), g.misc = F(IN_MISC);
    g.q2k = I(IN_Q2K), g.tok2q = I(IN_TOK2Q), g.q2ta = I(IN_Q2TA);
    g.chir_w = F(IN_CHIR_W), g.chir_a = F(IN_CHIR_A), g.chir_c = I(IN_CHIR_C), g.chir_ptr = I(IN_CHIR_PTR), g.chir_idx = I(IN_CHIR_IDX);
    auto BF = [&](int b) { return reinterpret_cast<float*>(ws + t.off[b]); };
    auto BH = [&](int b) { return reinterpret_cast<bf16*>(ws + t.off[b]); };
    Bufs& b = p.buf;
    b.pos = BF(B_POS), b.xn = BF(B_XN), b.out = BF(B_OUT), b.cen = BF(B_CEN), b.ntv = BF(B_NTV), b.sc = BF(B_SC);
    b.se = BF(B_SE), b.qa = BF(B_QA), b.skip = BF(B_SKIP), b.act = BF(B_ACT), b.tb = BF(B_TB), b.upd = BF(B_UPD);
    b.agt = BF(B_AGT), b.grad = BF(B_GRAD), b.kab = BF(B_KAB);
    b.sct = BH(B_SCT), b.scln0 = BH(B_SCLN0), b.scbf = BH(B_SCBF), b.sch = BH(B_SCH), b.mods = BH(B_MODS);
    b.ao = BH(B_AO), b.abf = BH(B_ABF), b.aqg = BH(B_AQG), b.akv = BH(B_AKV), b.tx = BH(B_TX), b.qkvg = BH(B_QKVG);
    b.to = BH(B_TO), b.tc = BH(B_TC), b.plg = BH(B_PLG), b.axq = BH(B_AXQ), b.axk = BH(B_AXK), b.axhl = BH(B_AXHL);
    b.aca = BH(B_ACA), b.vt = BH(B_VT), b.tx2 = t.flags & F_PARALLEL ? BH(B_TX2) : b.tx;
    p.flow_cnt = reinterpret_cast<unsigned int*>(ws + t.off[B_FLOW]);
    p.ctl = reinterpret_cast<Control*>(ws);

    const size_t rt = size_t(t.S) * N, ra = size_t(t.S) * A, cs = t.cs;
    struct AMap {
        int id;
        const void* base;
        size_t rows, cols;
    } amaps[] = {
        {TM_A_SCT, b.sct, size_t(N), cs}, {TM_A_SCH, b.sch, size_t(N), 2 * cs}, {TM_A_SCLN0, b.scln0, size_t(N), cs},
        {TM_A_SCBF, b.scbf, size_t(N), cs}, {TM_A_TX, b.tx, rt, kTokC}, {TM_A_TX2, b.tx2, rt, kTokC}, {TM_A_TO, b.to, rt, kTokC},
        {TM_A_TC, b.tc, rt, kTokHidden}, {TM_A_ABF, b.abf, ra, kAtomC}, {TM_A_AXQ, b.axq, ra, kAtomC},
        {TM_A_AXK, b.axk, ra, kAtomC}, {TM_A_AO, b.ao, ra, kAtomC}, {TM_A_AXHL, b.axhl, ra, 2 * kAtomC},
        {TM_A_ACA, b.aca, ra, kAtomHidden}, {TM_A_PC, in[IN_PC], size_t(N) * N, size_t(t.plc)},
    };
    for (const AMap& m : amaps) {
        if (int e = encode_map(&L.tmap[m.id], m.base, m.rows, m.cols, m.cols, kBM)) {
            return e;
        }
    }
    // token attention: Q/K tiles of QKVG (64 columns x 64 rows), VT tiles (64 keys x 48 dims), bias tiles
    if (int e = encode_map(&L.tmap[TM_T_QK], b.qkvg, rt, kQKVG, kQKVG, 64)) {
        return e;
    }
    if (int e = encode_map(&L.tmap[TM_T_VT], b.vt, size_t(t.S) * kTokC, size_t(t.np), size_t(t.np), kHeadD)) {
        return e;
    }
    if (int e = encode_map(&L.tmap[TM_T_PLG], b.plg, size_t(t.nb) * kPairHeads * t.np, size_t(t.np), size_t(t.np), 128)) {
        return e;
    }
    // the attention's output: a softmax warp's 32 rows of one head
    if (int e = encode_rows_store_map(&L.tmap[TM_T_TO], b.to, rt, kTokC, 32, kHeadD)) {
        return e;
    }
    const size_t nb = t.nb;
    struct OMap {
        int id;
        const void* base;
        size_t rows, cols;
    } omaps[] = {
        {TM_O_QKVG, b.qkvg, rt, kQKVG}, {TM_O_AQG, b.aqg, ra, 2 * kAtomC}, {TM_O_AKV, b.akv, ra, 2 * kAtomC},
        {TM_O_TC, b.tc, rt, kTokHidden}, {TM_O_ACA, b.aca, ra, kAtomHidden}, {TM_O_SCH, b.sch, size_t(N), 2 * cs},
        {TM_O_MODS, b.mods, nb * kTokModSlots * N, kTokC},
    };
    for (const OMap& m : omaps) {
        if (int e = encode_store_map(&L.tmap[m.id], m.base, m.rows, m.cols)) {
            return e;
        }
    }
    struct BMap {
        int id, in;
        size_t rows, cols, m; // m: rows of the GEMM's A, for the tile choice
        int n;                // the GEMM's n (per block)
        int max_bn = kMaxBN;  // gated-residual epilogues hold a whole tile's inputs in registers
        int unit = 64;        // GLU GEMMs: rows of W1 per unit
    } bmaps[] = {
        {TM_B_ST0_W1, IN_ST0_W1, 4 * cs, cs, size_t(N), int(4 * cs)}, {TM_B_ST1_W1, IN_ST1_W1, 4 * cs, cs, size_t(N), int(4 * cs)},
        {TM_B_ST0_W2, IN_ST0_W2, cs, 2 * cs, size_t(N), int(cs)}, {TM_B_ST1_W2, IN_ST1_W2, cs, 2 * cs, size_t(N), int(cs)},
        {TM_B_WM1, IN_WM1, nb * kTokMods1 * kTokC, cs, size_t(N), int(nb * kTokMods1 * kTokC)},
        {TM_B_WM2, IN_WM2, nb * 2 * kTokC, cs, size_t(N), int(nb * 2 * kTokC)},
        {TM_B_WSE, IN_WSE, kTokC, cs, size_t(N), kTokC},
        {TM_B_WQKVG, IN_WQKVG, nb * kQKVG, kTokC, rt, kQKVG}, {TM_B_WO, IN_WO, nb * kTokC, kTokC, rt, kTokC, kResidMaxBnBf},
        {TM_B_W1, IN_W1, nb * t.tw1, kTokC, rt, t.tw1, kMaxBN, t.tw1 / (kTokHidden / kGluHalf)}, {TM_B_W2, IN_W2, nb * kTokC, kTokHidden, rt, kTokC, kResidMaxBnBf},
        {TM_B_WTB, IN_WTB, kAtomC, kTokC, rt, kAtomC}, {TM_B_WAGGR, IN_WAGGR, kTokC, kAtomC, ra, kTokC},
        {TM_B_PLW, IN_PLW, nb * kPairHeads, size_t(t.plc), size_t(N) * N, int(nb * kPairHeads)},
        {TM_B_ENC_WQG, IN_ENC_WQG, 3 * 2 * kAtomC, kAtomC, ra, 2 * kAtomC}, {TM_B_ENC_WKV, IN_ENC_WKV, 3 * 2 * kAtomC, kAtomC, ra, 2 * kAtomC},
        {TM_B_ENC_WO, IN_ENC_WO, 3 * kAtomC, kAtomC, ra, kAtomC, kResidMaxBnF32}, {TM_B_ENC_W1, IN_ENC_W1, size_t(3 * t.aw1), kAtomC, ra, t.aw1, kMaxBN, t.aw1 / (kAtomHidden / kGluHalf)},
        {TM_B_ENC_W2, IN_ENC_W2, 3 * kAtomC, kAtomHidden, ra, kAtomC, kResidMaxBnF32},
        {TM_B_DEC_WQG, IN_DEC_WQG, 3 * 2 * kAtomC, kAtomC, ra, 2 * kAtomC}, {TM_B_DEC_WKV, IN_DEC_WKV, 3 * 2 * kAtomC, kAtomC, ra, 2 * kAtomC},
        {TM_B_DEC_WO, IN_DEC_WO, 3 * kAtomC, kAtomC, ra, kAtomC, kResidMaxBnF32}, {TM_B_DEC_W1, IN_DEC_W1, size_t(3 * t.aw1), kAtomC, ra, t.aw1, kMaxBN, t.aw1 / (kAtomHidden / kGluHalf)},
        {TM_B_DEC_W2, IN_DEC_W2, 3 * kAtomC, kAtomHidden, ra, kAtomC, kResidMaxBnF32},
    };
    for (const BMap& m : bmaps) {
        const int bn = choose_bn(m.m, m.n, dev.sms, m.max_bn, m.unit);
        p.bn[m.id] = bn;
        if (int e = encode_map(&L.tmap[m.id], in[m.in], m.rows, m.cols, m.cols, bn)) {
            return e;
        }
    }
    return make_program(L.prog, 0, t.nsteps, t.flags | (p.flow ? kProgFlow : 0));
}

// control words zeroed | the persistent kernel: two stream operations, no host synchronisation
static int enqueue(const Launch& L, const Device& dev, cudaStream_t st) {
    if (cudaMemsetAsync(L.kp.ctl, 0, sizeof(Control), st) != cudaSuccess) {
        return fail(E_LAUNCH, std::string("MkSample: ") + cudaGetErrorString(cudaGetLastError()));
    }
    void* args[] = {const_cast<Launch*>(&L)};
    const cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(cck_sampler_kernel), dim3(dev.sms),
                                                        dim3(kThreads), args, kSmemAlloc, st);
    if (err != cudaSuccess) {
        return fail(E_LAUNCH, std::string("MkSample: ") + cudaGetErrorString(err));
    }
    return E_OK;
}

} // namespace cck

// The dense GEMM engine: C = A·Wᵀ with bf16 operands and f32 accumulation on the 5th-generation
// tensor cores. Per CTA: one thread feeds a 4-stage shared-memory ring with TMA tile loads, one
// thread issues tcgen05.mma into a double-buffered TMEM accumulator (2 x 256 columns), and four
// warps drain finished accumulators with tcgen05.ld and apply the fused epilogue, so the epilogue
// of tile i overlaps the main loop of tile i+1. Tiles are 128 x bn (bn = 64..256) x 64.
//
// The epilogue kinds restate the reference's (src/diffusion/gemm.cuh:156-325) on a
// one-thread-per-row accumulator layout.
#pragma once

#ifndef CCK_EPI_DB
#define CCK_EPI_DB 0
#endif
// CCK_STAGE_REC=1 builds a diagnostics variant: every CTA stamps the moments of its roles inside a
// phase (first TMA issued, first operands landed, last MMA issued, last accumulator seen, epilogue
// done, barrier reached, barrier left) and the sums per phase kind are read with mk_stage_rec
#ifndef CCK_STAGE_REC
#define CCK_STAGE_REC 0
#endif

#include "params.cuh"
#include "ptx.cuh"

namespace cck {

constexpr int kBM = 128, kBK = 64, kStages = 4, kMaxBN = 256;
constexpr int kStageA = kBM * kBK * 2;        // 16 KB
constexpr int kStageB = kMaxBN * kBK * 2;     // 32 KB
constexpr int kStageBytes = kStageA + kStageB;
constexpr int kPipeBytes = kStages * kStageBytes; // 192 KB
constexpr int kTmemCols = 512;
// Warp roles in the tensor-core phases: warp 0 holds the TMA thread, warp 1 the MMA thread, warps
// 2..9 are the workers that read TMEM (accumulator epilogues, attention softmax). A warp may only
// touch the TMEM lanes 32·(warp % 4).., so the eight workers form two groups of four, each group
// covering all 128 lanes; the groups split a tile's columns between them.
// Two more warps follow the workers: in the token attention, which runs two pipelines per CTA, they
// hold the second pipeline's TMA and MMA threads; in GEMM phases they have no role.
constexpr int kWorkWarp0 = 2, kWorkWarps = 8, kAuxWarp0 = kWorkWarp0 + kWorkWarps;
static_assert(kAuxWarp0 + 2 == kWarps, "TMA, MMA, eight workers (two per TMEM lane quarter), and the second pipeline's TMA and MMA");
constexpr int kAttnItemWarps = 4; // softmax warps that store the rows of one token-attention item (one group of workers)
__device__ __forceinline__ int work_quarter() {
    return warp_id() & 3;
}
__device__ __forceinline__ int work_group() {
    return (warp_id() - kWorkWarp0) >> 2;
}

// shared-memory control block
struct SmemCtl {
    uint64_t full[kStages], empty[kStages]; // TMA -> MMA, MMA -> TMA
    uint64_t tfull[2], tempty[2];           // MMA -> epilogue, epilogue -> MMA
    uint32_t tmem_base;
    volatile int abort;
    volatile int quit;                      // the launch has failed somewhere: leave the schedule
    unsigned long long t0;                  // end of the previous phase, ns (timing record, CTA 0)
#if CCK_STAGE_REC
    unsigned long long stamp[16], phase_t0;
#endif
};
#if CCK_STAGE_REC
__device__ unsigned long long g_stage_rec[32][16];
// SM clock cycles: cheap to read, comparable within one CTA
__device__ __forceinline__ unsigned long long stage_now() {
    return (unsigned long long)clock64();
}
#define CCK_STAMP(i, first_only)                                                          \
    do {                                                                                  \
        SmemCtl* c_ = smem_ctl();                                                         \
        if (!(first_only) || c_->stamp[i] == 0) c_->stamp[i] = stage_now();               \
    } while (0)
#else
#define CCK_STAMP(i, first_only) do { } while (0)
#endif

// CCK_TRACE=n builds another diagnostics variant: threads of CTA n - 1 write (cycle, event, value)
// records of what they pass, each role into its own 2048 slots (no atomics, one store per event), over
// the phases of a launch; mk_trace reads and clears them. Roles: 0, 1 the TMA threads; 2, 3 the MMA
// threads; 4, 5 the first worker thread of each group (token attention: per pipeline); 6 thread 0
// between the operations (operation begins, ends, grid barrier reached, passed).
// Events: 0x10.. TMA, 0x20.. MMA, 0x30.. softmax of the token attention (+1: second pipeline);
// 0x50.. TMA, 0x60.. MMA, 0x70.. epilogue of a GEMM; 0x80.. the schedule.
#ifndef CCK_TRACE
#define CCK_TRACE 0
#endif
#if CCK_TRACE
constexpr int kTraceRoles = 7, kTraceSlots = 2048;
__device__ unsigned long long g_trace[kTraceRoles][kTraceSlots];
__device__ unsigned int g_trace_n[kTraceRoles];
constexpr int kBarWaitSlots = 1024;
__device__ unsigned int g_barwait[kBarWaitSlots][160]; // [grid barrier][CTA]: cycles waited | phase kind << 24
#define CCK_TRACE_BEGIN_IF(role, cond) \
    const int tr_role_ = (role);       \
    unsigned int tr_n_ = (blockIdx.x == CCK_TRACE - 1 && (cond)) ? g_trace_n[tr_role_] : 0xffffffffu
#define CCK_TRACE_BEGIN(role) CCK_TRACE_BEGIN_IF(role, true)
#define CCK_TRACE_EV(code, val)                                                                                  \
    do {                                                                                                         \
        if (tr_n_ < kTraceSlots) {                                                                               \
            g_trace[tr_role_][tr_n_++] = (unsigned long long)(clock64()) << 16 | (unsigned long long)((code) << 8 | ((val) & 255)); \
        }                                                                                                        \
    } while (0)
#define CCK_TRACE_END()                                        \
    do {                                                       \
        if (tr_n_ != 0xffffffffu) g_trace_n[tr_role_] = tr_n_; \
    } while (0)
#define CCK_TRACE_ONE(role, code, val) \
    do {                               \
        CCK_TRACE_BEGIN(role);         \
        CCK_TRACE_EV(code, val);       \
        CCK_TRACE_END();               \
    } while (0)
#else
#define CCK_TRACE_BEGIN_IF(role, cond) do { } while (0)
#define CCK_TRACE_BEGIN(role) do { } while (0)
#define CCK_TRACE_EV(code, val) do { } while (0)
#define CCK_TRACE_END() do { } while (0)
#define CCK_TRACE_ONE(role, code, val) do { } while (0)
#endif

static_assert(sizeof(SmemCtl) <= 256, "SmemCtl outgrew its part of the control block");
// Shared memory of the CTA: [pipeline stages | epilogue stages | control | schedule state | the
// parameter block | GEMM descriptors]. The first two are contiguous: phases without a GEMM use
// them as one scratch area.
constexpr int kEpiStageBytes = 32 * 16 * 4;                     // per worker warp: 32 rows x 16 floats
constexpr int kEpiOff = kPipeBytes;
constexpr int kScratchBytes = kPipeBytes + kWorkWarps * kEpiStageBytes;
constexpr int kCtlOff = kScratchBytes;                          // SmemCtl, the timing record, the attention barriers
constexpr int kTimingOff = 256, kTcBarsOff = 640;               // in the control block: per-kind [ns, phases] of the timing record; the attention barriers
static_assert(kTimingOff + 2 * kKinds * 8 <= kTcBarsOff, "the control block's parts overlap");
constexpr int kRunSlot = 24;                                    // bytes of per-thread schedule state (Run)
constexpr int kCtlBytes = 1280;
constexpr int kRunOff = kCtlOff + kCtlBytes;
constexpr int kKpOff = kRunOff + kRunSlot * kThreads;           // the CTA's copy of the parameter block
constexpr int kKpBytes = 1280;
constexpr int kGdOff = kKpOff + kKpBytes;                       // prepared GEMM descriptors
constexpr int kGdBytes = 4608;
constexpr int kProgOff = kGdOff + kGdBytes;                     // the phase program
constexpr int kProgBytes = 512;
static_assert(sizeof(Program) <= kProgBytes, "the phase program outgrew its shared-memory slot");
constexpr int kBiasOff = kProgOff + kProgBytes;                 // per worker warp: the bias of one 32-column unit
constexpr int kSmemBytes = kBiasOff + kWorkWarps * 128;
static_assert(sizeof(KP) <= kKpBytes, "KP outgrew its shared-memory slot");
constexpr int kSmemAlloc = kSmemBytes + 1024;                   // slack to align the base to 1024 bytes
static_assert(kSmemAlloc <= 232448, "more than the 227 KB a CTA may have");

__device__ __forceinline__ char* smem_base() {
    extern __shared__ char smem_raw[];
    const uint32_t a = smem_u32(smem_raw);
    return smem_raw + ((1024u - (a & 1023u)) & 1023u);
}
// The parameter block with the call's real extents filled in (the kernel parameter holds the
// bucket's): every CTA keeps a copy in shared memory
__device__ __forceinline__ const KP& kp() {
    return *reinterpret_cast<const KP*>(smem_base() + kKpOff);
}
__device__ __forceinline__ SmemCtl* smem_ctl() {
    return reinterpret_cast<SmemCtl*>(smem_base() + kCtlOff);
}
__device__ __forceinline__ long long wait_limit() {
    return kp().wait_cycles;
}
// Records the launch's first failure and tells the grid: the poison bit in the barrier word ends
// every CTA's wait at its next barrier (sampler.cuh: grid_barrier), after which the schedule is left.
__device__ __forceinline__ void fail_launch(unsigned int code, unsigned int where) {
    Control* c = kp().ctl;
    if (atomicCAS(&c->status, ST_OK, code) == ST_OK) {
        c->where = where;
    }
    atomicOr(&c->barrier, kBarrierPoison);
}

// per-thread pipeline positions, kept across phases for the whole launch
struct Pipe {
    uint32_t kb = 0;   // k-blocks produced (TMA thread) or consumed (MMA thread)
    uint32_t tile = 0; // accumulator tiles issued (MMA thread) or drained (worker threads)
};

// Work dealing: item i of a phase goes to CTA (start + i) mod grid, and consecutive work lists of
// one phase continue the rotation (as the reference's Deal, src/diffusion/gemm.cuh:84-95)
struct Deal {
    int start = 0;
    __device__ int first() const {
        return (int(blockIdx.x) - start + int(gridDim.x)) % int(gridDim.x);
    }
    __device__ void advance(int items) {
        start = (start + items) % int(gridDim.x);
    }
};

__host__ __device__ inline int cdiv(int a, int b) {
    return (a + b - 1) / b;
}

// ---- epilogues
// An accumulator tile leaves TMEM with one row per lane. Global memory wants the opposite:
// consecutive lanes on consecutive columns of one row. So each worker warp turns 32 rows x 16
// columns at a time through a private shared-memory stage (64-byte rows, 16-byte pieces XOR-swizzled:
// conflict-free both ways), after which lane l holds the four columns 4(l % 4).. of rows l / 4 + 8i,
// i < 4: every warp access covers eight full 64-byte row segments.
constexpr int kPiece = 16;
__device__ __forceinline__ float* epi_stage() {
    return reinterpret_cast<float*>(smem_base() + kEpiOff + (warp_id() - kWorkWarp0) * kEpiStageBytes);
}
// row-per-lane values v[16 pc .. 16 pc + 15] -> column-per-lane t[i] (row l / 4 + 8i)
template <int PC> __device__ __forceinline__ void epi_turn(float* st, const float (&v)[32], float4 (&t)[4]) {
    const int l = lane_id();
    float4* w = reinterpret_cast<float4*>(st + l * kPiece);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        w[i ^ ((l >> 1) & 3)] = make_float4(v[16 * PC + 4 * i], v[16 * PC + 4 * i + 1], v[16 * PC + 4 * i + 2], v[16 * PC + 4 * i + 3]);
    }
    __syncwarp();
    const int r = l >> 2, c = l & 3;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = r + 8 * i;
        t[i] = *reinterpret_cast<const float4*>(st + row * kPiece + 4 * (c ^ ((row >> 1) & 3)));
    }
    __syncwarp();
}
__device__ __forceinline__ uint2 pack_bf4(float4 x) {
    return make_uint2(pack_bf2(x.x, x.y), pack_bf2(x.z, x.w));
}
__device__ __forceinline__ float4 unpack_bf4(uint2 u) {
    return make_float4(bf_to_f32(u.x & 0xFFFFu), bf_to_f32(u.x >> 16), bf_to_f32(u.y & 0xFFFFu), bf_to_f32(u.y >> 16));
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ float4 sigmoid4(float4 x) {
    return make_float4(sigmoid_fast(x.x), sigmoid_fast(x.y), sigmoid_fast(x.z), sigmoid_fast(x.w));
}

// What a unit of 32 columns needs from global memory besides the accumulator: the bias of its two
// pieces, fetched one unit ahead (the first unit's before the accumulator is complete), because
// after a grid barrier every such load is an L2 round trip
struct EpiPre {
    float4 b[2];
};
template <int E> __device__ __forceinline__ void epi_prefetch(const GemmDesc& g, int c0, EpiPre& pre) {
    if constexpr (E == EPI_BF16 || E == EPI_F32 || E == EPI_MODS) {
        const int col = c0 + 4 * (lane_id() & 3);
#pragma unroll
        for (int pc = 0; pc < 2; pc++) {
            pre.b[pc] = g.bias && col + kPiece * pc < g.bias_cols ? *reinterpret_cast<const float4*>(g.bias + col + kPiece * pc)
                                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}
// per unit: where its rows go (row r of the GEMM at o + r·ld, in elements of the output type) and
// whether the sigmoid applies
struct EpiUnit {
    void* o;
    int ld;
    bool sig;
};
template <int E> __device__ __forceinline__ EpiUnit epi_unit(const GemmDesc& g, int oc) {
    EpiUnit u;
    u.ld = g.ldo, u.sig = false;
    if constexpr (E == EPI_MODS) {
        // column c is slot slot0 + (c / 768) % slots of block c / (slots·768): one slot per unit
        const int blk = oc / (g.slots * kTokC), slot = g.slot0 + (oc / kTokC) % g.slots;
        u.sig = g.sig_slots >> slot & 1;
        u.o = static_cast<bf16*>(g.out) + (size_t(blk) * kTokModSlots + slot) * g.period * kTokC + oc % kTokC;
        u.ld = kTokC;
    } else if constexpr (E == EPI_BF16 || E == EPI_GLU) {
        u.sig = oc >= g.sig_from;
        u.o = static_cast<bf16*>(g.out) + oc;
    } else {
        u.o = static_cast<float*>(g.out) + oc;
    }
    return u;
}

// one piece after the turn: rows r0 + 8i, columns c..c+3 of the unit
template <int E> __device__ __forceinline__ void epi_store(const GemmDesc& g, const EpiUnit& u, int r0, int c, const float4 (&t)[4],
                                                           const float4& b) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = r0 + 8 * i;
        if (row >= g.m) {
            continue;
        }
        if constexpr (E == EPI_BF16 || E == EPI_MODS || E == EPI_GLU) {
            float4 x = E == EPI_GLU ? t[i] : add4(t[i], b);
            if (E != EPI_GLU && u.sig) {
                x = sigmoid4(x);
            }
            *reinterpret_cast<uint2*>(static_cast<bf16*>(u.o) + size_t(row) * u.ld + c) = pack_bf4(x);
        } else if constexpr (E == EPI_F32) {
            float4 x = add4(t[i], b);
            if (g.relu) {
                x = make_float4(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f), fmaxf(x.z, 0.f), fmaxf(x.w, 0.f));
            }
            *reinterpret_cast<float4*>(static_cast<float*>(u.o) + size_t(row) * u.ld + c) = x;
        } else if constexpr (E == EPI_SCRES) {
            float4* o = reinterpret_cast<float4*>(static_cast<float*>(u.o) + size_t(row) * u.ld + c);
            *o = add4(*o, t[i]);
        }
    }
}

// The pair logits of one unit: a tile's rows are 128 consecutive keys k of one query q (rbase
// encodes q·ktiles·128 + k0), the column is the table (block·16 + head); base-2 logits. Lanes are
// consecutive k of one table row already: stored without the turn. Keys past the real tokens are
// masked, keys past the padded extent are not stored.
__device__ __forceinline__ void pair_unit(const GemmDesc& g, int rbase, int c0, const float (&v)[32]) {
    const int q = rbase / (g.ktiles * kBM), k = rbase % (g.ktiles * kBM) + lane_id();
    if (q < g.nreal && k < g.npreal) {
        const TokenW& tw = kp().tw;
        const bool masked = k >= g.nreal || tw.tmask[k] == 0.f;
        const size_t pq = size_t(q) * g.ldn + (masked ? 0 : k);
        const float mean = tw.pcs[2 * pq], rstd = tw.pcs[2 * pq + 1];
        const float extra = kp().plx ? bf_to_f32(tw.plx[pq]) : 0.f;
        bf16* o = static_cast<bf16*>(g.out) + size_t(q) * g.np + k;
        const size_t plane = size_t(g.np) * g.np;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const int col = c0 + i;
            const float y = kLog2e * (masked ? -kMaskBias : rstd * (v[i] - mean * tw.plws[col]) + tw.plb[col] + extra);
            o[col * plane] = bf16(pack_bf2(y, 0.f) & 0xFFFFu);
        }
    }
}
// the v columns of QKVG, transposed: lanes are consecutive tokens, column hd of 32 tokens is one
// 64-byte run of VT
__device__ __forceinline__ void vt_unit(const GemmDesc& g, int rbase, int c0, const float (&v)[32]) {
    const int row = rbase + lane_id();
    if (row < g.m) {
        bf16* o = g.vt + (size_t(row / g.period) * kTokC + (c0 - 2 * kTokC)) * g.np + row % g.period;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            o[size_t(i) * g.np] = bf16(pack_bf2(v[i], 0.f) & 0xFFFFu);
        }
    }
}

// A unit of bf16 output through TMA: the warp's 32 rows x 32 columns go row-per-lane (as they
// leave TMEM) into the warp's stage in the 64-byte-swizzled layout of the store map, and one lane
// issues the store. No turn, no per-row address arithmetic; rows past the tensor's end are clipped
// by the copy, so the caller takes this path only when all 32 rows belong to the GEMM.
__device__ __forceinline__ void store_unit_tma(const CUtensorMap* mo, float* st, int x, int y, const float (&v)[32]) {
    const int l = lane_id();
    if (l == 0) {
        bulk_wait_read(); // the previous store has read the stage
    }
    __syncwarp();
    uint4* row = reinterpret_cast<uint4*>(reinterpret_cast<char*>(st) + 64 * l);
#pragma unroll
    for (int c = 0; c < 4; c++) {
        row[c ^ ((l >> 1) & 3)] = make_uint4(pack_bf2(v[8 * c], v[8 * c + 1]), pack_bf2(v[8 * c + 2], v[8 * c + 3]),
                                            pack_bf2(v[8 * c + 4], v[8 * c + 5]), pack_bf2(v[8 * c + 6], v[8 * c + 7]));
    }
    fence_async_smem();
    __syncwarp();
    if (l == 0) {
        tma_store_2d(mo, x, y, st);
        bulk_commit();
    }
}

// The epilogue of one 128 x bn accumulator held in TMEM columns [acc, acc + bn), by the eight
// worker warps: units of 32 output columns alternate between the two groups. Waits for the
// accumulator itself, after the first unit's global loads are under way.
template <int E> __device__ __forceinline__ void epilogue_tile(const GemmDesc& g, const CUtensorMap* mo, uint32_t acc, int row0, int col0,
                                                               uint64_t* tfull, uint32_t tpar, volatile int* abort) {
    const int q = work_quarter(), gp = work_group();
    const int rbase = row0 + q * 32, r0 = rbase + (lane_id() >> 2), cl = 4 * (lane_id() & 3);
    const uint32_t taddr = acc + (uint32_t(q * 32) << 16);
    float* st = epi_stage();
    const int kIn = E == EPI_GLU ? g.glu_unit : 32; // accumulator columns per unit
    constexpr bool kTma = E == EPI_BF16 || E == EPI_GLU || E == EPI_MODS;
    const int units = g.bn / kIn;
    // output column of unit u: a GLU unit of 64 (or 96) columns gives 32
    const int oc0 = E == EPI_GLU ? col0 / kIn * kGluHalf : col0;
    if constexpr (kTma) {
        if (mo && rbase + 32 <= g.m) {
            // ---- all 32 rows are real: TMA stores. The unit's bias (one value per lane) waits in the
            // warp's shared-memory slot, fetched a unit ahead.
            float* bs = reinterpret_cast<float*>(smem_base() + kBiasOff) + (warp_id() - kWorkWarp0) * 32;
            const bool has_bias = E != EPI_GLU && g.bias != nullptr;
            float bnext = 0.f;
            if (has_bias && gp < units) {
                const int c = oc0 + 32 * gp + lane_id();
                bnext = c < g.bias_cols ? g.bias[c] : 0.f;
            }
            mbar_wait(tfull, tpar, abort);
            if (threadIdx.x == kWorkWarp0 * 32) {
                CCK_STAMP(3, false);
            }
            tc_fence_after();
#pragma unroll 1
            for (int u = gp; u < units; u += 2) {
                const int oc = oc0 + 32 * u;
                if (has_bias) {
                    __syncwarp();
                    bs[lane_id()] = bnext;
                    __syncwarp();
                    if (u + 2 < units) {
                        const int c = oc + 64 + lane_id();
                        bnext = c < g.bias_cols ? g.bias[c] : 0.f;
                    }
                }
                float v[32];
                if constexpr (E == EPI_GLU) {
                    uint32_t ga[32], pr[32];
                    tmem_ld32_issue(taddr + u * kIn, ga);
                    tmem_ld32_issue(taddr + u * kIn + kGluHalf, pr);
                    tmem_ld_wait(ga);
                    tmem_ld_wait(pr);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        v[i] = silu_fast(__uint_as_float(ga[i])) * __uint_as_float(pr[i]);
                    }
                    if (kIn > 2 * kGluHalf) { // [gate | proj | a_to_b]: the third part multiplies
                        float ab[32];
                        tmem_ld32(taddr + u * kIn + 2 * kGluHalf, ab);
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            v[i] *= ab[i];
                        }
                    }
                } else {
                    tmem_ld32(taddr + u * kIn, v);
                }
                if (has_bias) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float4 bb = reinterpret_cast<const float4*>(bs)[i];
                        v[4 * i] += bb.x, v[4 * i + 1] += bb.y, v[4 * i + 2] += bb.z, v[4 * i + 3] += bb.w;
                    }
                }
                int x = oc, y = rbase;
                bool sig = false;
                if constexpr (E == EPI_BF16) {
                    sig = oc >= g.sig_from;
                    if (g.vt && oc >= 2 * kTokC && oc < 3 * kTokC) {
                        vt_unit(g, rbase, oc, v);
                    }
                }
                if constexpr (E == EPI_MODS) {
                    // column c is slot slot0 + (c / 768) % slots of block c / (slots·768): one slot per unit
                    const int blk = oc / (g.slots * kTokC), slot = g.slot0 + (oc / kTokC) % g.slots;
                    sig = g.sig_slots >> slot & 1;
                    x = oc % kTokC, y = (blk * kTokModSlots + slot) * g.period + rbase;
                }
                if (sig) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        v[i] = sigmoid_fast(v[i]);
                    }
                }
                store_unit_tma(mo, st, x, y, v);
            }
            return;
        }
        if (lane_id() == 0) {
            bulk_wait_read(); // a store of an earlier tile may still be reading the stage
        }
        __syncwarp();
    }
    EpiPre cur, nxt;
    if (gp < units) {
        epi_prefetch<E>(g, oc0 + 32 * gp, cur);
    }
    mbar_wait(tfull, tpar, abort);
    if (threadIdx.x == kWorkWarp0 * 32) {
        CCK_STAMP(3, false);
    }
    tc_fence_after();
#pragma unroll 1
    for (int u = gp; u < units; u += 2) {
        const int oc = oc0 + 32 * u;
        if (u + 2 < units) {
            epi_prefetch<E>(g, oc + 64, nxt);
        }
        float v[32];
        if constexpr (E == EPI_GLU) {
            // [gate 32 | proj 32] per unit of 64 accumulator columns -> 32 outputs
            uint32_t ga[32], pr[32];
            tmem_ld32_issue(taddr + u * kIn, ga);
            tmem_ld32_issue(taddr + u * kIn + kGluHalf, pr);
            tmem_ld_wait(ga);
            tmem_ld_wait(pr);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                v[i] = silu_fast(__uint_as_float(ga[i])) * __uint_as_float(pr[i]);
            }
            if (kIn > 2 * kGluHalf) {
                float ab[32];
                tmem_ld32(taddr + u * kIn + 2 * kGluHalf, ab);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    v[i] *= ab[i];
                }
            }
        } else {
            tmem_ld32(taddr + u * kIn, v);
        }
        if constexpr (E == EPI_PAIR) {
            pair_unit(g, rbase, oc, v);
        } else {
            if constexpr (E == EPI_BF16) {
                if (g.vt && oc >= 2 * kTokC && oc < 3 * kTokC) {
                    vt_unit(g, rbase, oc, v);
                }
            }
            const EpiUnit eu = epi_unit<E>(g, oc);
            float4 t[4];
            epi_turn<0>(st, v, t);
            epi_store<E>(g, eu, r0, cl, t, cur.b[0]);
            epi_turn<1>(st, v, t);
            epi_store<E>(g, eu, r0, kPiece + cl, t, cur.b[1]);
        }
        cur = nxt;
    }
}

// The gated residual update out = src + gate ⊙ C · rowmask. Everything it reads besides the
// accumulator depends on addresses only, so it is fetched while the main loop runs: the residual
// rows by cp.async into shared memory that the pipeline leaves free (these GEMMs have bn <= 128, so
// the upper 16 KB of each stage's 32 KB weight slot is unused; each worker warp owns 8 KB of it,
// 16 slots of 16 bytes per lane), the gates into registers (bf16) or beside the residual (f32,
// bn <= 64).
constexpr int kResidMaxBnBf = 128, kResidMaxBnF32 = 64;
__device__ __forceinline__ void cp_async16_cg(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.wait_all;" ::: "memory");
}
template <bool GF32>
__device__ __forceinline__ void resid_tile(const GemmDesc& g, uint32_t acc, int row0, int col0, uint64_t* tfull, uint32_t tpar,
                                           volatile int* abort) {
    constexpr int kU = GF32 ? 1 : 2; // units of 32 columns per warp
    const int q = work_quarter(), gp = work_group(), ww = warp_id() - kWorkWarp0;
    const int r0 = row0 + q * 32 + (lane_id() >> 2), cl = 4 * (lane_id() & 3);
    const uint32_t taddr = acc + (uint32_t(q * 32) << 16);
    float4* area = reinterpret_cast<float4*>(smem_base() + (ww >> 1) * kStageBytes + kStageA + kStageB / 2 + (ww & 1) * 8192) + lane_id();
    const float* src = static_cast<const float*>(g.out);
    const int units = g.bn / 32;
    float m[4];
    const bf16* gp4[4]; // bf16 gates: this lane's four rows at the tile's first column
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = min(r0 + 8 * i, g.m - 1), p = row % g.period;
        m[i] = g.rowmask ? g.rowmask[p] : 1.f;
        const float* sp = src + size_t(row) * g.ldo + col0 + cl;
        const size_t go = size_t(p) * g.ldg + col0 + cl;
        gp4[i] = static_cast<const bf16*>(g.gate) + go;
#pragma unroll
        for (int k = 0; k < kU; k++) {
            const int u = gp + 2 * k;
            if (u < units) {
#pragma unroll
                for (int pc = 0; pc < 2; pc++) {
                    const int c = 32 * u + kPiece * pc, slot = (k * 2 + pc) * 4 + i;
                    cp_async16_cg(area + slot * 32, sp + c);
                    if constexpr (GF32) {
                        cp_async16_cg(area + (8 + slot) * 32, static_cast<const float*>(g.gate) + go + c);
                    }
                }
            }
        }
    }
    // bf16 gates travel in registers, one piece ahead of their use
    uint2 gcur[4], gnxt[4];
    if constexpr (!GF32) {
        if (gp < units) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                gcur[i] = *reinterpret_cast<const uint2*>(gp4[i] + 32 * gp);
            }
        }
    }
    mbar_wait(tfull, tpar, abort);
    if (threadIdx.x == kWorkWarp0 * 32) {
        CCK_STAMP(3, false);
    }
    tc_fence_after();
    cp_async_wait_all();
    float* st = epi_stage();
    float* op = static_cast<float*>(g.out) + col0 + cl;
#pragma unroll
    for (int k = 0; k < kU; k++) {
        const int u = gp + 2 * k;
        if (u < units) {
#pragma unroll
            for (int pc = 0; pc < 2; pc++) {
                const int c = 32 * u + kPiece * pc;
                if constexpr (!GF32) {
                    // the next piece of this warp: the unit's second piece, or the next unit's first
                    const int cn = pc == 0 ? c + kPiece : c + 64 - kPiece;
                    if (pc == 0 || u + 2 < units) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            gnxt[i] = *reinterpret_cast<const uint2*>(gp4[i] + cn);
                        }
                    }
                }
                float v[32]; // one piece: the first 16 are used
                {
                    float h[16];
                    tmem_ld16(taddr + c, h);
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        v[i] = h[i];
                    }
                }
                float4 t[4];
                epi_turn<0>(st, v, t);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int row = r0 + 8 * i;
                    if (row < g.m) {
                        const int slot = (k * 2 + pc) * 4 + i;
                        const float4 x = area[slot * 32];
                        float4 gt;
                        if constexpr (GF32) {
                            gt = area[(8 + slot) * 32];
                        } else {
                            gt = unpack_bf4(gcur[i]);
                        }
                        const float4 cc = t[i];
                        *reinterpret_cast<float4*>(op + size_t(row) * g.ldo + c) =
                            make_float4(x.x + gt.x * cc.x * m[i], x.y + gt.y * cc.y * m[i], x.z + gt.z * cc.z * m[i], x.w + gt.w * cc.w * m[i]);
                    }
                }
                if constexpr (!GF32) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        gcur[i] = gnxt[i];
                    }
                }
            }
        }
    }
    // What this warp read and wrote here with ordinary accesses (its staging area inside the pipeline
    // stages, the turn through its epilogue stage) is shared memory that later TMA loads overwrite:
    // order the two proxies.
    fence_async_smem();
}

// tile t -> (row tile, column tile) without an integer division
__device__ __forceinline__ void tile_coords(const GemmDesc& g, int t, int& row0, int& col0) {
    // t = major · inner + minor: (column tile, row tile) with inner = mt, or with nfast (row tile,
    // column tile) with inner = nt: a row tile's column tiles are dealt together, its rows complete early
    const int inner = (g.fl & GF_NFAST) ? g.nt : g.mt;
    const int major = g.mt_magic ? int(__umulhi((unsigned int)t, g.mt_magic)) : t / inner, minor = t - major * inner;
    row0 = ((g.fl & GF_NFAST) ? major : minor) * kBM, col0 = ((g.fl & GF_NFAST) ? minor : major) * g.bn;
}
__host__ __device__ inline void gd_finish(GemmDesc& g) {
    g.nt = g.n / g.bn;
    g.mt = cdiv(g.m, kBM), g.tiles = g.mt * g.nt;
    const int inner = (g.fl & GF_NFAST) ? g.nt : g.mt;
    // exact while t · inner < 2^32; otherwise 0: divide
    g.mt_magic = (unsigned long long)(g.tiles) * inner < 0x100000000ull ? (unsigned int)((0x100000000ull + inner - 1) / inner) : 0u;
    if (inner == 1) {
        g.mt_magic = 0; // 2^32 does not fit
    }
}

// ---- prepared GEMM descriptors: built once per launch into shared memory, so that a phase starts
// with a few shared-memory loads instead of a few hundred dependent scalar instructions
__device__ __forceinline__ GemmDesc* gd_table() {
    return reinterpret_cast<GemmDesc*>(smem_base() + kGdOff);
}
constexpr int kMaxGd = kGdBytes / int(sizeof(GemmDesc));

// ---- completion counters between operations of one phase (FlowCnt)
__device__ __forceinline__ unsigned int* flow_cnt(const KP& p, int which) {
    return p.flow_cnt + which * p.flow_n;
}
// The calling warp's part of a unit is stored: its lanes' writes (and lane 0's TMA stores, which the
// caller has waited for) are published with one release add per counter in [c0, c1].
__device__ __forceinline__ void flow_signal(unsigned int* cnt, int c0, int c1) {
    fence_async_global(); // ordinary stores, for TMA reads in other CTAs
    __syncwarp();
    if (lane_id() == 0) {
        for (int c = c0; c <= c1; c++) {
            red_release_add(cnt + c, 1u);
        }
    }
}
// One thread waits until the counters [c0, c1] have reached target (bounded, as every wait here);
// what it then reads through TMA is what the signalling warps wrote. The counters are read eight at
// a time with relaxed loads (one L2 round trip for the batch, not one each) and one acquire fence
// follows the last read.
__device__ __forceinline__ bool flow_wait(const unsigned int* cnt, int c0, int c1, unsigned int target, volatile int* abort) {
    const long long t0 = clock64();
    unsigned int* status = &kp().ctl->status;
    if (*abort) { // a wait inside this CTA gave up earlier: tell the grid, which would otherwise wait for this CTA's units
        fail_launch(ST_PIPE_TIMEOUT, 0);
    }
    for (int b0 = c0; b0 <= c1; b0 += 8) {
        for (;;) {
            unsigned int v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[i] = b0 + i <= c1 ? ld_relaxed(cnt + b0 + i) : target;
            }
            bool ok = true;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                ok = ok && v[i] >= target;
            }
            if (ok) {
                break;
            }
            if (*abort) {
                return false;
            }
            // another CTA gave up (its units will not come), or this wait ran out: the launch drains
            if (ld_relaxed(status) != ST_OK || clock64() - t0 > wait_limit()) {
                fail_launch(ST_PIPE_TIMEOUT, 0);
                *abort = 1;
                return false;
            }
            __nanosleep(20);
        }
    }
    fence_acq_rel_gpu();
    fence_async_global();
    return true;
}
// Arrivals that complete row block rb of a GEMM's A (descriptor g, depc set) in one token block. TO:
// the attention items of every block of 128 queries (per sample of g.period rows) that the rows
// touch, 16 heads x 4 warps each. TC: the column tiles of W1 over these rows, 8 warps each. TX: the
// adaLN rows of the block.
__device__ __forceinline__ unsigned int flow_target(const GemmDesc& g, int which, int rb, int w1_tiles) {
    if (which == FC_TX) {
        return (unsigned int)(min(kBM, g.m - rb * kBM));
    }
    if (which != FC_TO) {
        return (unsigned int)(w1_tiles * kWorkWarps);
    }
    const int lo = rb * kBM, hi = min(lo + kBM, g.m) - 1, qblocks = cdiv(g.period, kBM);
    const int ilo = lo / g.period * qblocks + lo % g.period / kBM, ihi = hi / g.period * qblocks + hi % g.period / kBM;
    return (unsigned int)(kHeads * kAttnItemWarps * (ihi - ilo + 1));
}

// the worker warps' loop over the tiles of one GEMM, block b of its stack; every finished tile is
// reported to the completion counter of its block of 128 rows, if the descriptor names one
template <int E> __device__ CCK_HOT_FN void worker_tiles(const GemmDesc& gd, const CUtensorMap* mo, int b, uint32_t tile, int tb, int te, int ts,
                                                         unsigned int epoch) {
    SmemCtl* ctl = smem_ctl();
    GemmDesc g = gd; // a private copy: stores through its pointers cannot alias it
    g.bias = g.bias ? g.bias + size_t(b) * g.bias_step : nullptr;
    g.gate = static_cast<const char*>(g.gate) + (long long)(b)*g.gate_step;
    CCK_TRACE_BEGIN_IF(4, threadIdx.x == kWorkWarp0 * 32);
    CCK_TRACE_EV(0x70, E);
    for (int t = tb; t < te; t += ts, tile++) {
        int row0, col0;
        tile_coords(gd, t, row0, col0); // (from the shared-memory descriptor: nothing of it held across the epilogue)
        const uint32_t buf = tile & 1, tpar = (tile >> 1) & 1;
        const uint32_t acc = ctl->tmem_base + buf * kMaxBN;
        if constexpr (E == EPI_RESID) {
            // The epilogue fetches the residual rows ahead, under the main loop. Where the operation that
            // wrote them last shares this phase (W2: the rows come from WO, no barrier since), they are
            // final once the tile's own dependency is met: WO's tiles over the rows came before the adaLN
            // rows, W1's tiles and so the counter that the tile's TMA thread waits for as well.
            if ((gd.fl >> GF_DEP_SHIFT & GF_CNT_MASK) == 1 + FC_TC) {
                if (lane_id() == 0) {
                    flow_wait(flow_cnt(kp(), FC_TC), row0 / kBM, row0 / kBM, (epoch + 1) * flow_target(gd, FC_TC, row0 / kBM, gd_table()[GD_TOK_W1].nt),
                              &ctl->abort);
                }
                __syncwarp();
            }
            if (g.gate_f32) {
                resid_tile<true>(g, acc, row0, col0, &ctl->tfull[buf], tpar, &ctl->abort);
            } else {
                resid_tile<false>(g, acc, row0, col0, &ctl->tfull[buf], tpar, &ctl->abort);
            }
        } else {
            epilogue_tile<E>(g, mo, acc, row0, col0, &ctl->tfull[buf], tpar, &ctl->abort);
        }
        tc_fence_before();
        __syncwarp();
        CCK_TRACE_EV(0x72, t); // the accumulator is read
        if (lane_id() == 0) {
            mbar_arrive(&ctl->tempty[buf]);
            if (warp_id() == kWorkWarp0) {
                CCK_STAMP(4, false);
            }
        }
        if constexpr (E == EPI_BF16 || E == EPI_GLU || E == EPI_RESID) {
            if (const int sigc = gd.fl >> GF_SIG_SHIFT & GF_CNT_MASK) {
                if (E != EPI_RESID && lane_id() == 0) {
                    bulk_wait_done();
                }
                int r0, c0; // (recomputed: not held across the epilogue)
                tile_coords(gd, t, r0, c0);
                flow_signal(flow_cnt(kp(), sigc - 1), r0 / kBM, r0 / kBM);
            }
        }
        CCK_TRACE_EV(0x74, t); // stored and reported
    }
    if constexpr (E == EPI_BF16 || E == EPI_GLU || E == EPI_MODS) {
        if (lane_id() == 0) {
            bulk_wait_done(); // this warp's TMA stores have landed before the phase ends
        }
        __syncwarp();
    }
    CCK_TRACE_EV(0x76, 0);
    CCK_TRACE_END();
}

// ---- the TMA and MMA roles over the tiles of one GEMM
// Tiles tb, tb + ts, ... < te (tile t: rows (t % mt)·128, columns (t / mt)·bn) of descriptor gd
// with block b of its stack applied; one thread each.
// k-blocks [kb0, kb1) of tile t into the ring, from position kbc on
__device__ __forceinline__ void produce_kblocks(const Launch& L, const GemmDesc& gd, int b, int t, int kb0, int kb1, uint32_t& kbc) {
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    const CUtensorMap* ma = &L.tmap[gd.map_a];
    const CUtensorMap* mb = &L.tmap[gd.map_b];
    const int ktiles = gd.ktiles, kwrap = gd.b_kwrap;
    const uint32_t bytes = kStageA + uint32_t(gd.bn) * kBK * 2;
    int row0, col0;
    tile_coords(gd, t, row0, col0);
    // pair GEMM: row tile (q, key tile) starts at row q·ldn + k0 of PC
    const int arow = ktiles ? row0 / (ktiles * kBM) * gd.ldn + row0 % (ktiles * kBM) : gd.a_row0 + row0;
    const int brow = gd.b_row0 + b * gd.b_step + col0;
    for (int kb = kb0; kb < kb1; kb++, kbc++) {
        const uint32_t s = kbc % kStages, par = (kbc / kStages) & 1;
        mbar_wait(&ctl->empty[s], par ^ 1, &ctl->abort);
        CCK_STAMP(10, true);
        mbar_expect_tx(&ctl->full[s], bytes);
        char* st = sm + s * kStageBytes;
        const int ka = kb * kBK, kw = kwrap ? ka % kwrap : ka;
        tma_load_2d(st, ma, ka, arow, &ctl->full[s]);
        tma_load_2d(st + kStageA, mb, kw, brow, &ctl->full[s]);
        CCK_STAMP(0, true);
    }
}
// The TMA role over this CTA's tiles of one GEMM. After a grid barrier the thread that saw the
// barrier open runs it right there for the phase's first GEMM (ahead = true), before the rest of
// the CTA has found its way to the operation: the ramp of the phase (operation fetch, role
// dispatch) then runs under the loads' latency. pipe.tile of the producer thread (otherwise unused)
// says that the next call has nothing left to do.
__device__ CCK_PHASE_FN void gemm_produce(const Launch& L, Pipe& pipe, const GemmDesc& gd, int b, int tb, int te, int ts, bool ahead,
                                          unsigned int epoch) {
    if (pipe.tile) { // produced ahead
        pipe.tile = 0;
        return;
    }
    const int kblocks = gd.k / kBK;
    uint32_t kbc = pipe.kb;
    CCK_TRACE_BEGIN(0);
    CCK_TRACE_EV(0x50, gd.epi);
    for (int t = tb; t < te; t += ts) {
        if (const int depc = gd.fl >> GF_DEP_SHIFT & GF_CNT_MASK) { // until the rows of A that this tile reads are complete
            int row0, col0;
            tile_coords(gd, t, row0, col0);
            const int rb = row0 / kBM;
#if CCK_STAGE_REC
            const long long fw0_ = clock64();
#endif
            flow_wait(flow_cnt(kp(), depc - 1), rb, rb, (epoch + 1) * flow_target(gd, depc - 1, rb, gd_table()[GD_TOK_W1].nt),
                      &smem_ctl()->abort);
#if CCK_STAGE_REC
            atomicAdd(&g_stage_rec[28][3 + (depc - 1)], (unsigned long long)(clock64() - fw0_)); // row 28: 4 waits for TO, 5 waits for TC
            atomicAdd(&g_stage_rec[28][6 + (depc - 1)], 1ull);                                  // 7, 8: how many
#endif
        }
        CCK_TRACE_EV(0x52, t); // what the tile reads is complete
        produce_kblocks(L, gd, b, t, 0, kblocks, kbc);
        CCK_TRACE_EV(0x54, t); // every k-block is asked for
    }
    CCK_TRACE_END();
    pipe.kb = kbc;
    pipe.tile = ahead;
}
__device__ CCK_PHASE_FN void gemm_issue(Pipe& pipe, const GemmDesc& gd, int tb, int te, int ts) {
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    const int bn = gd.bn, kblocks = gd.k / kBK;
    const uint32_t idesc = umma_idesc_bf16(kBM, bn);
    uint32_t kbc = pipe.kb, tile = pipe.tile;
    CCK_TRACE_BEGIN(2);
    CCK_TRACE_EV(0x60, gd.epi);
    for (int t = tb; t < te; t += ts, tile++) {
        const uint32_t buf = tile & 1, tpar = (tile >> 1) & 1;
        mbar_wait(&ctl->tempty[buf], tpar ^ 1, &ctl->abort);
        tc_fence_after();
        CCK_TRACE_EV(0x62, t); // the accumulator buffer is free
        const uint32_t acc = ctl->tmem_base + buf * kMaxBN;
        for (int kb = 0; kb < kblocks; kb++, kbc++) {
            const uint32_t s = kbc % kStages, par = (kbc / kStages) & 1;
            mbar_wait(&ctl->full[s], par, &ctl->abort);
            CCK_STAMP(1, true);
            tc_fence_after();
            if (kb == 0) {
                CCK_TRACE_EV(0x64, t); // the first operands have landed
            }
            const uint32_t sa = smem_u32(sm + s * kStageBytes), sb = sa + kStageA;
            const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; kk++) {
                // 16 bf16 = 32 bytes along k inside the 128-byte swizzle row: +2 in the address field
                umma_bf16(acc, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
            }
            umma_commit(&ctl->empty[s]);
        }
        umma_commit(&ctl->tfull[buf]);
        CCK_STAMP(2, false);
        CCK_TRACE_EV(0x66, t); // the tile's last MMA is issued
    }
    CCK_TRACE_END();
    pipe.kb = kbc, pipe.tile = tile;
}

// once per launch, by the whole CTA: barriers and the TMEM allocation
__device__ inline void gemm_init() {
    SmemCtl* ctl = smem_ctl();
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(&ctl->full[i], 1);
            mbar_init(&ctl->empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&ctl->tfull[i], 1);
            mbar_init(&ctl->tempty[i], kWorkWarps);
        }
        ctl->abort = 0, ctl->quit = 0;
        ctl->t0 = 0;
        fence_mbar_init();
    }
    if (warp_id() == 0) {
        tmem_alloc(&ctl->tmem_base, kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
}
__device__ inline void gemm_fini() {
    tc_fence_before();
    __syncthreads();
    if (warp_id() == 0) {
        tmem_dealloc(smem_ctl()->tmem_base, kTmemCols);
    }
}

} // namespace cck

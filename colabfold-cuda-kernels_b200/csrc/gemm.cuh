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
constexpr int kEpiWarp0 = 4; // warps 4..7 drain TMEM lanes 0..127

// shared-memory control block, placed after the pipeline stages
struct SmemCtl {
    uint64_t full[kStages], empty[kStages]; // TMA -> MMA, MMA -> TMA
    uint64_t tfull[2], tempty[2];           // MMA -> epilogue, epilogue -> MMA
    uint64_t aux[8];                        // attention phases
    uint32_t tmem_base;
    volatile int abort;
#if CCK_STAGE_REC
    unsigned long long stamp[16], phase_t0;
#endif
};
#if CCK_STAGE_REC
__device__ unsigned long long g_stage_rec[32][16];
__device__ __forceinline__ unsigned long long stage_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define CCK_STAMP(i, first_only)                                                          \
    do {                                                                                  \
        SmemCtl* c_ = reinterpret_cast<SmemCtl*>(smem_base() + kPipeBytes);               \
        if (!(first_only) || c_->stamp[i] == 0) c_->stamp[i] = stage_now();               \
    } while (0)
#else
#define CCK_STAMP(i, first_only) do { } while (0)
#endif
constexpr int kRunSlot = 48;                                    // bytes of per-thread schedule state (Run)
constexpr int kRunOff = kPipeBytes + 1024 + 4 * 32 * 36 * 4;    // it follows the epilogue stages
constexpr int kKpOff = kRunOff + kRunSlot * kThreads;           // the CTA's copy of the parameter block
constexpr int kSmemBytes = kKpOff + 1024;                       // stages, control, epilogue stages, run state, KP
static_assert(sizeof(KP) <= 1024, "KP outgrew its shared-memory slot");
constexpr int kSmemAlloc = kSmemBytes + 1024;                   // slack to align the base to 1024 bytes

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
    return reinterpret_cast<SmemCtl*>(smem_base() + kPipeBytes);
}

// per-thread pipeline positions, kept across phases for the whole launch
struct Pipe {
    uint32_t kb = 0;   // k-blocks produced (TMA thread) or consumed (MMA thread)
    uint32_t tile = 0; // accumulator tiles issued (MMA thread) or drained (epilogue threads)
};

// Work dealing: item i of a phase goes to CTA (start + i) mod grid, and consecutive work lists of
// one phase continue the rotation (as the reference's Deal, src/diffusion/gemm.cuh:84-95)
struct Deal {
    int start = 0;
    bool live = true;
    __device__ int first() const {
        return live ? (int(blockIdx.x) - start + int(gridDim.x)) % int(gridDim.x) : (1 << 28);
    }
    __device__ void advance(int items) {
        start = (start + items) % int(gridDim.x);
    }
};

__host__ __device__ inline int cdiv(int a, int b) {
    return (a + b - 1) / b;
}

// ---- epilogues
// An accumulator tile leaves TMEM with one row per lane (32 lanes x 32 columns per load). Global
// memory wants the opposite: consecutive lanes on consecutive columns of one row. So each epilogue
// warp turns its 32 x 32 block around through a private shared-memory stage (rows of 36 floats:
// conflict-free 16-byte accesses both ways), after which lane l handles the four columns
// 4(l % 8).. of rows l / 8 + 4i, i < 8: every warp access covers four full 128-byte row segments.
constexpr int kEpiPitch = 36;                         // floats per staged row
constexpr int kEpiStageFloats = 32 * kEpiPitch;       // per epilogue warp
constexpr int kEpiStageBytes = 4 * kEpiStageFloats * 4;

__device__ __forceinline__ float* epi_stage() {
    return reinterpret_cast<float*>(smem_base() + kPipeBytes + 1024) + (warp_id() & 3) * kEpiStageFloats;
}
// row-per-lane registers -> the stage -> column-per-lane registers (piece i: row l / 8 + 4i)
__device__ __forceinline__ void epi_turn(float* st, const float (&v)[32], float4 (&t)[8]) {
    float4* w = reinterpret_cast<float4*>(st + lane_id() * kEpiPitch);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        w[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
    __syncwarp();
    const int r = lane_id() >> 3, cj = lane_id() & 7;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        t[i] = *reinterpret_cast<const float4*>(st + (r + 4 * i) * kEpiPitch + 4 * cj);
    }
    __syncwarp();
}
__device__ __forceinline__ uint2 pack_bf4(float4 x) {
    return make_uint2(pack_bf2(x.x, x.y), pack_bf2(x.z, x.w));
}
__device__ __forceinline__ float4 unpack_bf4(uint2 u) {
    return make_float4(bf_to_f32(u.x & 0xFFFFu), bf_to_f32(u.x >> 16), bf_to_f32(u.y & 0xFFFFu), bf_to_f32(u.y >> 16));
}

// one 32-column chunk, columns c0.. of the GEMM, rows rbase.. of the GEMM (this warp's 32 rows)
template <int E> __device__ __forceinline__ void epi_chunk(const GemmDesc& g, float* st, int rbase, int c0, float (&v)[32]) {
    if constexpr (E == EPI_PAIR) {
        // A tile's rows are 128 consecutive keys k of one query q (rbase encodes q·ktiles·128 + k0),
        // the column is the table (block·16 + head); base-2 logits. Lanes are consecutive k of one
        // table row already: stored without the turn. Keys past the real tokens are masked, keys
        // past the padded extent are not stored.
        const int q = rbase / (g.ktiles * kBM), k = rbase % (g.ktiles * kBM) + lane_id();
        if (q < g.nreal && k < g.npreal) {
            const bool masked = k >= g.nreal || g.tmask[k] == 0.f;
            const size_t pq = size_t(q) * g.ldn + (masked ? 0 : k);
            const float mean = g.pcs[2 * pq], rstd = g.pcs[2 * pq + 1];
            const float extra = g.plx ? bf_to_f32(g.plx[pq]) : 0.f;
            bf16* o = static_cast<bf16*>(g.out) + size_t(q) * g.np + k;
            const size_t plane = size_t(g.np) * g.np;
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const int col = c0 + i;
                const float y = kLog2e * (masked ? -kMaskBias : rstd * (v[i] - mean * g.plws[col]) + g.plb[col] + extra);
                o[col * plane] = bf16(pack_bf2(y, 0.f) & 0xFFFFu);
            }
        }
        return;
    }
    if constexpr (E == EPI_BF16) {
        if (g.vt && c0 >= 2 * kTokC && c0 < 3 * kTokC) {
            // lanes are consecutive tokens here: column hd of 32 tokens is one 64-byte run of VT
            const int row = rbase + lane_id();
            if (row < g.m) {
                bf16* o = g.vt + (size_t(row / g.period) * kTokC + (c0 - 2 * kTokC)) * g.np + row % g.period;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    o[size_t(i) * g.np] = bf16(pack_bf2(v[i], 0.f) & 0xFFFFu);
                }
            }
        }
    }
    float4 t[8];
    epi_turn(st, v, t);
    const int r0 = rbase + (lane_id() >> 3), col = c0 + 4 * (lane_id() & 7);
    if constexpr (E == EPI_BF16) {
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g.bias && col < g.bias_cols) {
            b = *reinterpret_cast<const float4*>(g.bias + col);
        }
        const bool sig = col >= g.sig_from;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = r0 + 4 * i;
            float4 x = make_float4(t[i].x + b.x, t[i].y + b.y, t[i].z + b.z, t[i].w + b.w);
            if (sig) {
                x = make_float4(sigmoid_fast(x.x), sigmoid_fast(x.y), sigmoid_fast(x.z), sigmoid_fast(x.w));
            }
            if (row < g.m) {
                *reinterpret_cast<uint2*>(static_cast<bf16*>(g.out) + size_t(row) * g.ldo + col) = pack_bf4(x);
            }
        }
    } else if constexpr (E == EPI_GLU) {
        // v already holds silu(gate)·proj of one unit; its 32 outputs start at column c0
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = r0 + 4 * i;
            if (row < g.m) {
                *reinterpret_cast<uint2*>(static_cast<bf16*>(g.out) + size_t(row) * g.ldo + col) = pack_bf4(t[i]);
            }
        }
    } else if constexpr (E == EPI_F32) {
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g.bias) {
            b = *reinterpret_cast<const float4*>(g.bias + col);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = r0 + 4 * i;
            float4 x = make_float4(t[i].x + b.x, t[i].y + b.y, t[i].z + b.z, t[i].w + b.w);
            if (g.relu) {
                x = make_float4(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f), fmaxf(x.z, 0.f), fmaxf(x.w, 0.f));
            }
            if (row < g.m) {
                *reinterpret_cast<float4*>(static_cast<float*>(g.out) + size_t(row) * g.ldo + col) = x;
            }
        }
    } else if constexpr (E == EPI_SCRES) {
        float4 in[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = min(r0 + 4 * i, g.m - 1);
            in[i] = *reinterpret_cast<const float4*>(static_cast<const float*>(g.out) + size_t(row) * g.ldo + col);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = r0 + 4 * i;
            if (row < g.m) {
                *reinterpret_cast<float4*>(static_cast<float*>(g.out) + size_t(row) * g.ldo + col) =
                    make_float4(in[i].x + t[i].x, in[i].y + t[i].y, in[i].z + t[i].z, in[i].w + t[i].w);
            }
        }
    } else if constexpr (E == EPI_RESID) {
        // handled by resid_load / resid_apply
    } else if constexpr (E == EPI_MODS) {
        // column c is slot slot0 + (c / 768) % slots of block c / (slots·768)
        const int blk = c0 / (g.slots * kTokC), slot = g.slot0 + (c0 / kTokC) % g.slots;
        const bool sig = g.sig_slots >> slot & 1;
        const float4 b = *reinterpret_cast<const float4*>(g.bias + col);
        bf16* o = static_cast<bf16*>(g.out) + (size_t(blk) * kTokModSlots + slot) * g.period * kTokC + col % kTokC;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int row = r0 + 4 * i;
            float4 x = make_float4(t[i].x + b.x, t[i].y + b.y, t[i].z + b.z, t[i].w + b.w);
            if (sig) {
                x = make_float4(sigmoid_fast(x.x), sigmoid_fast(x.y), sigmoid_fast(x.z), sigmoid_fast(x.w));
            }
            if (row < g.m) {
                *reinterpret_cast<uint2*>(o + size_t(row) * kTokC) = pack_bf4(x);
            }
        }
    }
}

// The gated residual update out = src + gate ⊙ C · rowmask in two halves: the loads of a chunk
// (residual, gate, row mask) depend on addresses only, so they are issued before the accumulator
// chunk is read out of TMEM, and the first chunk's even before the accumulator is complete.
struct ResidRegs {
    float4 in[8], gt[8];
    float m[8];
};
__device__ __forceinline__ void resid_load(const GemmDesc& g, int rbase, int c0, ResidRegs& rr) {
    const int r0 = rbase + (lane_id() >> 3), col = c0 + 4 * (lane_id() & 7);
    const float* src = g.src ? g.src : static_cast<const float*>(g.out);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = min(r0 + 4 * i, g.m - 1), p = row % g.period;
        rr.in[i] = *reinterpret_cast<const float4*>(src + size_t(row) * g.ldo + col);
        if (g.gate_f32) {
            rr.gt[i] = *reinterpret_cast<const float4*>(static_cast<const float*>(g.gate) + size_t(p) * g.ldg + col);
        } else {
            rr.gt[i] = unpack_bf4(*reinterpret_cast<const uint2*>(static_cast<const bf16*>(g.gate) + size_t(p) * g.ldg + col));
        }
        rr.m[i] = g.rowmask ? g.rowmask[p] : 1.f;
    }
}
__device__ __forceinline__ void resid_apply(const GemmDesc& g, float* st, int rbase, int c0, float (&v)[32], const ResidRegs& rr) {
    float4 t[8];
    epi_turn(st, v, t);
    const int r0 = rbase + (lane_id() >> 3), col = c0 + 4 * (lane_id() & 7);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = r0 + 4 * i;
        if (row < g.m) {
            const float m = rr.m[i];
            *reinterpret_cast<float4*>(static_cast<float*>(g.out) + size_t(row) * g.ldo + col) =
                make_float4(rr.in[i].x + rr.gt[i].x * t[i].x * m, rr.in[i].y + rr.gt[i].y * t[i].y * m,
                            rr.in[i].z + rr.gt[i].z * t[i].z * m, rr.in[i].w + rr.gt[i].w * t[i].w * m);
        }
    }
}
// the whole tile: waits for the accumulator itself
__device__ __forceinline__ void resid_tile(const GemmDesc& g, uint32_t acc, int row0, int col0, uint64_t* tfull, uint32_t tpar,
                                           volatile int* abort) {
    const int q = warp_id() & 3, rbase = row0 + q * 32;
    const uint32_t taddr = acc + (uint32_t(q * 32) << 16);
    float* st = epi_stage();
    ResidRegs rr;
    resid_load(g, rbase, col0, rr);
    mbar_wait(tfull, tpar, abort);
    if (threadIdx.x == kEpiWarp0 * 32) {
        CCK_STAMP(3, false);
    }
    tc_fence_after();
    for (int c = 0; c < g.bn; c += 32) {
        float v[32];
        tmem_ld32(taddr + c, v);
        resid_apply(g, st, rbase, col0 + c, v, rr);
        if (c + 32 < g.bn) {
            resid_load(g, rbase, col0 + c + 32, rr);
        }
    }
}

// the epilogue of one 128 x bn accumulator held in TMEM columns [acc, acc + bn)
template <int E> __device__ __forceinline__ void epilogue_tile(const GemmDesc& g, uint32_t acc, int row0, int col0) {
    const int q = warp_id() & 3;
    const int rbase = row0 + q * 32;
    const uint32_t taddr = acc + (uint32_t(q * 32) << 16);
    float* st = epi_stage();
    if constexpr (E == EPI_GLU) {
        // [gate 32 | proj 32] per unit of 64 columns -> 32 outputs
        for (int c = 0; c < g.bn; c += 2 * kGluHalf) {
            float gate[32], proj[32];
            tmem_ld32(taddr + c, gate);
            tmem_ld32(taddr + c + kGluHalf, proj);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                gate[i] = silu_fast(gate[i]) * proj[i];
            }
            epi_chunk<E>(g, st, rbase, (col0 + c) / 2, gate);
        }
    } else {
#if CCK_EPI_DB
        // two chunks of TMEM reads in flight: the next one is issued before this one is processed
        uint32_t ra[32], rb[32];
        tmem_ld32_issue(taddr, ra);
        for (int c = 0; c < g.bn; c += 64) {
            float v[32];
            tmem_ld_wait(ra);
            if (c + 32 < g.bn) {
                tmem_ld32_issue(taddr + c + 32, rb);
            }
#pragma unroll
            for (int i = 0; i < 32; i++) {
                v[i] = __uint_as_float(ra[i]);
            }
            epi_chunk<E>(g, st, rbase, col0 + c, v);
            if (c + 32 < g.bn) {
                tmem_ld_wait(rb);
                if (c + 64 < g.bn) {
                    tmem_ld32_issue(taddr + c + 64, ra);
                }
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    v[i] = __uint_as_float(rb[i]);
                }
                epi_chunk<E>(g, st, rbase, col0 + c + 32, v);
            }
        }
#else
        for (int c = 0; c < g.bn; c += 32) {
            float v[32];
            tmem_ld32(taddr + c, v);
            epi_chunk<E>(g, st, rbase, col0 + c, v);
        }
#endif
    }
}
__device__ __forceinline__ void epilogue_dispatch(const GemmDesc& g, uint32_t acc, int row0, int col0) {
    switch (g.epi) {
    case EPI_BF16:
        epilogue_tile<EPI_BF16>(g, acc, row0, col0);
        break;
    case EPI_F32:
        epilogue_tile<EPI_F32>(g, acc, row0, col0);
        break;
    case EPI_SCRES:
        epilogue_tile<EPI_SCRES>(g, acc, row0, col0);
        break;
    case EPI_MODS:
        epilogue_tile<EPI_MODS>(g, acc, row0, col0);
        break;
    case EPI_GLU:
        epilogue_tile<EPI_GLU>(g, acc, row0, col0);
        break;
    default:
        epilogue_tile<EPI_PAIR>(g, acc, row0, col0);
    }
}

// ---- the three roles over the tiles of a list of GEMMs
// The three roles over tiles tb, tb + ts, ... < te of one GEMM (tile t: rows (t % mt)·128, columns
// (t / mt)·bn). Every thread of the CTA calls it with the same arguments.
__device__ __noinline__ void gemm_tiles(const Launch& L, Pipe& pipe, const GemmDesc& gd, int tb, int te, int ts) {
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    const int warp = warp_id(), lane = lane_id();
    if (threadIdx.x == 0) {
        CCK_STAMP(9, true);
    }
    const GemmDesc g = gd; // a private copy: stores through its pointers cannot alias it
    const int mt = cdiv(g.m, kBM), kblocks = g.k / kBK;
    if (warp == 0 && lane == 0) {
        // TMA producer
        const CUtensorMap* ma = &L.tmap[g.map_a];
        const CUtensorMap* mb = &L.tmap[g.map_b];
        const uint32_t bytes = kStageA + uint32_t(g.bn) * kBK * 2;
        for (int t = tb; t < te; t += ts) {
            const int row0 = t % mt * kBM, col0 = t / mt * g.bn;
            // pair GEMM: row tile (q, key tile) starts at row q·ldn + k0 of PC
            const int arow = g.ktiles ? row0 / (g.ktiles * kBM) * g.ldn + row0 % (g.ktiles * kBM) : g.a_row0 + row0;
            for (int kb = 0; kb < kblocks; kb++, pipe.kb++) {
                const uint32_t s = pipe.kb % kStages, par = (pipe.kb / kStages) & 1;
                mbar_wait(&ctl->empty[s], par ^ 1, &ctl->abort);
                CCK_STAMP(10, true);
                mbar_expect_tx(&ctl->full[s], bytes);
                char* st = sm + s * kStageBytes;
                const int ka = kb * kBK, kw = g.b_kwrap ? ka % g.b_kwrap : ka;
                tma_load_2d(st, ma, ka, arow, &ctl->full[s]);
                tma_load_2d(st + kStageA, mb, kw, g.b_row0 + col0, &ctl->full[s]);
                CCK_STAMP(0, true);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // MMA issuer
        const uint32_t idesc = umma_idesc_bf16(kBM, g.bn);
        for (int t = tb; t < te; t += ts, pipe.tile++) {
            const uint32_t buf = pipe.tile & 1, tpar = (pipe.tile >> 1) & 1;
            mbar_wait(&ctl->tempty[buf], tpar ^ 1, &ctl->abort);
            tc_fence_after();
            const uint32_t acc = ctl->tmem_base + buf * kMaxBN;
            for (int kb = 0; kb < kblocks; kb++, pipe.kb++) {
                const uint32_t s = pipe.kb % kStages, par = (pipe.kb / kStages) & 1;
                mbar_wait(&ctl->full[s], par, &ctl->abort);
                CCK_STAMP(1, true);
                tc_fence_after();
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
        }
    } else if (warp >= kEpiWarp0) {
        for (int t = tb; t < te; t += ts, pipe.tile++) {
            const int row0 = t % mt * kBM, col0 = t / mt * g.bn;
            const uint32_t buf = pipe.tile & 1, tpar = (pipe.tile >> 1) & 1;
            if (g.epi == EPI_RESID) {
                resid_tile(g, ctl->tmem_base + buf * kMaxBN, row0, col0, &ctl->tfull[buf], tpar, &ctl->abort);
            } else {
                mbar_wait(&ctl->tfull[buf], tpar, &ctl->abort);
                if (threadIdx.x == kEpiWarp0 * 32) {
                    CCK_STAMP(3, false);
                }
                tc_fence_after();
                epilogue_dispatch(g, ctl->tmem_base + buf * kMaxBN, row0, col0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->tempty[buf]);
                if (warp == kEpiWarp0) {
                    CCK_STAMP(4, false);
                }
            }
        }
    }
}
__device__ __forceinline__ int gemm_tile_count(const GemmDesc& g) {
    return cdiv(g.m, kBM) * (g.n / g.bn);
}
// a list of GEMMs whose tiles are dealt round-robin over the grid
__device__ inline void gemm_phase(const Launch& L, Pipe& pipe, Deal& d, const GemmDesc* list, int count) {
    for (int gi = 0; gi < count; gi++) {
        const int tiles = gemm_tile_count(list[gi]);
        gemm_tiles(L, pipe, list[gi], d.first(), tiles, gridDim.x);
        d.advance(tiles);
    }
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
            mbar_init(&ctl->tempty[i], kWarps - kEpiWarp0);
        }
        for (int i = 0; i < 8; i++) {
            mbar_init(&ctl->aux[i], 1);
        }
        ctl->abort = 0;
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

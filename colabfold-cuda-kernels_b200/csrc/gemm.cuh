// The dense GEMM engine: C = A·Wᵀ with bf16 operands and f32 accumulation on the 5th-generation
// tensor cores. Per CTA: one thread feeds a 4-stage shared-memory ring with TMA tile loads, one
// thread issues tcgen05.mma into a double-buffered TMEM accumulator (2 x 256 columns), and four
// warps drain finished accumulators with tcgen05.ld and apply the fused epilogue, so the epilogue
// of tile i overlaps the main loop of tile i+1. Tiles are 128 x bn (bn = 64..256) x 64.
//
// The epilogue kinds restate the reference's (src/diffusion/gemm.cuh:156-325) on a
// one-thread-per-row accumulator layout.
#pragma once

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
};
constexpr int kSmemBytes = kPipeBytes + 1024; // control block in the last KB
constexpr int kSmemAlloc = kSmemBytes + 1024; // slack to align the base to 1024 bytes

__device__ __forceinline__ char* smem_base() {
    extern __shared__ char smem_raw[];
    const uint32_t a = smem_u32(smem_raw);
    return smem_raw + ((1024u - (a & 1023u)) & 1023u);
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

// ---- epilogues: thread owns row `row`, v holds columns c0..c0+31 of the accumulator

__device__ __forceinline__ void store_bf32(bf16* dst, const float (&v)[32]) {
    uint4* p = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        p[i] = make_uint4(pack_bf2(v[8 * i], v[8 * i + 1]), pack_bf2(v[8 * i + 2], v[8 * i + 3]),
                          pack_bf2(v[8 * i + 4], v[8 * i + 5]), pack_bf2(v[8 * i + 6], v[8 * i + 7]));
    }
}

__device__ __forceinline__ void epi_chunk(const GemmDesc& g, int row, int c0, float (&v)[32]) {
    switch (g.epi) {
    case EPI_BF16:
    case EPI_QKVG: {
        if (g.bias && c0 < g.bias_cols) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
                v[i] += g.bias[c0 + i];
            }
        }
        if (c0 >= g.sig_from) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
                v[i] = sigmoid_fast(v[i]);
            }
        }
        store_bf32(static_cast<bf16*>(g.out) + size_t(row) * g.ldo + c0, v);
        if (g.epi == EPI_QKVG && c0 >= 2 * kTokC && c0 < 3 * kTokC) {
            // v also as [sample][head][d][np]: the K-major B operand of P·V
            const int s = row / g.period, tok = row % g.period;
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const int hd = c0 - 2 * kTokC + i;
                g.vt[(size_t(s) * kTokC + hd) * g.np + tok] = bf16(pack_bf2(v[i], 0.f) & 0xFFFFu);
            }
        }
        break;
    }
    case EPI_F32: {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(g.out) + size_t(row) * g.ldo + c0);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float4 x = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            if (g.bias) {
                const float4 b = *reinterpret_cast<const float4*>(g.bias + c0 + 4 * i);
                x.x += b.x, x.y += b.y, x.z += b.z, x.w += b.w;
            }
            if (g.relu) {
                x.x = fmaxf(x.x, 0.f), x.y = fmaxf(x.y, 0.f), x.z = fmaxf(x.z, 0.f), x.w = fmaxf(x.w, 0.f);
            }
            o[i] = x;
        }
        break;
    }
    case EPI_SCRES: {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(g.out) + size_t(row) * g.ldo + c0);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float4 x = o[i];
            x.x += v[4 * i], x.y += v[4 * i + 1], x.z += v[4 * i + 2], x.w += v[4 * i + 3];
            o[i] = x;
        }
        break;
    }
    case EPI_RESID: {
        const int p = row % g.period;
        const float m = g.rowmask ? g.rowmask[p] : 1.f;
        float gt[32];
        if (g.gate_f32) {
            const float4* gp = reinterpret_cast<const float4*>(static_cast<const float*>(g.gate) + size_t(p) * g.ldg + c0);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 x = gp[i];
                gt[4 * i] = x.x, gt[4 * i + 1] = x.y, gt[4 * i + 2] = x.z, gt[4 * i + 3] = x.w;
            }
        } else {
            const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const bf16*>(g.gate) + size_t(p) * g.ldg + c0);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 x = gp[i];
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    gt[8 * i + 2 * j] = bf_to_f32(w[j] & 0xFFFFu), gt[8 * i + 2 * j + 1] = bf_to_f32(w[j] >> 16);
                }
            }
        }
        float* of = static_cast<float*>(g.out) + size_t(row) * g.ldo + c0;
        const float4* in = reinterpret_cast<const float4*>(g.src ? g.src + size_t(row) * g.ldo + c0 : of);
        float4* o = reinterpret_cast<float4*>(of);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float4 x = in[i];
            float d0 = gt[4 * i] * v[4 * i], d1 = gt[4 * i + 1] * v[4 * i + 1];
            float d2 = gt[4 * i + 2] * v[4 * i + 2], d3 = gt[4 * i + 3] * v[4 * i + 3];
            if (g.rowmask) {
                d0 *= m, d1 *= m, d2 *= m, d3 *= m;
            }
            x.x += d0, x.y += d1, x.z += d2, x.w += d3;
            o[i] = x;
        }
        break;
    }
    case EPI_MODS: {
        // column c is slot slot0 + (c / 768) % slots of block c / (slots·768)
        const int blk = c0 / (g.slots * kTokC), slot = g.slot0 + (c0 / kTokC) % g.slots;
        const bool sig = g.sig_slots >> slot & 1;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            v[i] += g.bias[c0 + i];
            if (sig) {
                v[i] = sigmoid_fast(v[i]);
            }
        }
        store_bf32(static_cast<bf16*>(g.out) + ((size_t(blk) * kTokModSlots + slot) * g.period + row) * kTokC + c0 % kTokC, v);
        break;
    }
    case EPI_PAIR: {
        // row = pair (q, k) of the real tokens; column = table (block·16 + head); base-2 logits
        const int q = row / g.ldn, k = row % g.ldn;
        const bool masked = g.tmask[k] == 0.f;
        const size_t pq = size_t(q) * g.ldn + k;
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
        break;
    }
    default:
        break;
    }
}

// the epilogue of one 128 x bn accumulator held in TMEM columns [acc, acc + bn)
__device__ __forceinline__ void epilogue_tile(const GemmDesc& g, uint32_t acc, int row0, int col0) {
    const int q = warp_id() & 3;
    const int row = row0 + q * 32 + lane_id();
    const bool ok = row < g.m;
    const uint32_t taddr = acc + (uint32_t(q * 32) << 16);
    if (g.epi == EPI_GLU) {
        // [gate 32 | proj 32] per unit of 64 columns -> 32 outputs
        for (int c = 0; c < g.bn; c += 2 * kGluHalf) {
            float gate[32], proj[32];
            tmem_ld32(taddr + c, gate);
            tmem_ld32(taddr + c + kGluHalf, proj);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                gate[i] = silu_fast(gate[i]) * proj[i];
            }
            if (ok) {
                store_bf32(static_cast<bf16*>(g.out) + size_t(row) * g.ldo + (col0 + c) / 2, gate);
            }
        }
        return;
    }
    for (int c = 0; c < g.bn; c += 32) {
        float v[32];
        tmem_ld32(taddr + c, v);
        if (ok) {
            epi_chunk(g, row, col0 + c, v);
        }
    }
}

// ---- the three roles over the tiles of a list of GEMMs
__device__ __noinline__ void gemm_phase(const Launch& L, Pipe& pipe, Deal& d, const GemmDesc* list, int count) {
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    const int warp = warp_id(), lane = lane_id();
    for (int gi = 0; gi < count; gi++) {
        const GemmDesc& g = list[gi];
        const int mt = cdiv(g.m, kBM), tiles = mt * (g.n / g.bn), kblocks = g.k / kBK;
        const int t0 = d.first();
        if (warp == 0 && lane == 0) {
            // TMA producer
            const CUtensorMap* ma = &L.tmap[g.map_a];
            const CUtensorMap* mb = &L.tmap[g.map_b];
            const uint32_t bytes = kStageA + uint32_t(g.bn) * kBK * 2;
            for (int t = t0; t < tiles; t += gridDim.x) {
                const int row0 = t % mt * kBM, col0 = t / mt * g.bn;
                for (int kb = 0; kb < kblocks; kb++, pipe.kb++) {
                    const uint32_t s = pipe.kb % kStages, par = (pipe.kb / kStages) & 1;
                    mbar_wait(&ctl->empty[s], par ^ 1, &ctl->abort);
                    mbar_expect_tx(&ctl->full[s], bytes);
                    char* st = sm + s * kStageBytes;
                    const int ka = kb * kBK, kw = g.b_kwrap ? ka % g.b_kwrap : ka;
                    tma_load_2d(st, ma, ka, g.a_row0 + row0, &ctl->full[s]);
                    tma_load_2d(st + kStageA, mb, kw, g.b_row0 + col0, &ctl->full[s]);
                }
            }
        } else if (warp == 1 && lane == 0) {
            // MMA issuer
            const uint32_t idesc = umma_idesc_bf16(kBM, g.bn);
            for (int t = t0; t < tiles; t += gridDim.x, pipe.tile++) {
                const uint32_t buf = pipe.tile & 1, tpar = (pipe.tile >> 1) & 1;
                mbar_wait(&ctl->tempty[buf], tpar ^ 1, &ctl->abort);
                tc_fence_after();
                const uint32_t acc = ctl->tmem_base + buf * kMaxBN;
                for (int kb = 0; kb < kblocks; kb++, pipe.kb++) {
                    const uint32_t s = pipe.kb % kStages, par = (pipe.kb / kStages) & 1;
                    mbar_wait(&ctl->full[s], par, &ctl->abort);
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
            }
        } else if (warp >= kEpiWarp0) {
            for (int t = t0; t < tiles; t += gridDim.x, pipe.tile++) {
                const int row0 = t % mt * kBM, col0 = t / mt * g.bn;
                const uint32_t buf = pipe.tile & 1, tpar = (pipe.tile >> 1) & 1;
                mbar_wait(&ctl->tfull[buf], tpar, &ctl->abort);
                tc_fence_after();
                epilogue_tile(g, ctl->tmem_base + buf * kMaxBN, row0, col0);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&ctl->tempty[buf]);
                }
            }
        }
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

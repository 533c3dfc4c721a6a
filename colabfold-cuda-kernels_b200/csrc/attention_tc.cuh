// Token attention on the 5th-generation tensor cores: TO = softmax(q·kᵀ/√48 + L_b)·v ⊙ g.
//
// Item = (head, block of 128 queries, sample). Roles inside the CTA:
//   warp 0, one thread   TMA: the Q tile of the item (128 x 64 columns of QKVG at the head's q
//                        columns; 48 are used), then per chunk of 64 keys the K tile, the transposed
//                        V tile (48 x 64 from VT) and the 128 x 64 tile of pair logits, all with the
//                        128-byte swizzle, into a 4-deep ring
//   warp 1, one thread   tcgen05.mma: S = Q·Kᵀ (128 x 64, K = 48) into one of two TMEM buffers, and
//                        O_c = P·V (128 x 48, K = 64) with P read from shared memory
//   the 8 worker warps   two threads per query row (one per half of a chunk's keys and of the
//                        output dims): S out of TMEM, + bias, online base-2 softmax with the row
//                        maximum exchanged through shared memory, P (bf16) into shared memory in the
//                        swizzled K-major operand layout, the chunk's O_c out of TMEM into a register
//                        accumulator with the running rescale; finally o / l · gate -> TO
// So QKᵀ of chunk c+1 and P·V of chunk c-1 run on the tensor core while the softmax warps work on
// chunk c. Math as the reference's token attention (src/diffusion/attention.cuh:145-249): logits in
// base 2, P rounded to bf16 before P·V, row sums from the unrounded P.
#pragma once

#include "attention.cuh"

namespace cck {

constexpr int kTcKeys = 64;                     // keys per chunk
constexpr int kTcStages = 4;                    // ring depth of (K, Vt, bias) chunks
constexpr int kTcKBytes = kTcKeys * 128;        // 8 KB: 64 keys x 64 columns
constexpr int kTcVBytes = kHeadD * 128;         // 6 KB: 48 head dims x 64 keys
constexpr int kTcBiasBytes = 128 * 128;         // 16 KB: 128 queries x 64 keys
constexpr int kTcStageBytes = kTcKBytes + kTcVBytes + kTcBiasBytes; // 30 KB
constexpr int kTcQBytes = 128 * 128;            // 16 KB per Q buffer
constexpr int kTcPBytes = 128 * 128;            // 16 KB per P buffer
// shared memory: [ring 4 x 30 KB][Q x 2][P x 2] = 184 KB of the 192 KB pipeline area
constexpr int kTcQOff = kTcStages * kTcStageBytes, kTcPOff = kTcQOff + 2 * kTcQBytes;
constexpr int kTcXOff = kTcPOff + 2 * kTcPBytes; // 3 KB of row maxima and sums exchanged between the key halves
static_assert(kTcXOff + 3 * 1024 <= kPipeBytes, "the attention buffers live in the GEMM pipeline area");
// TMEM columns (the GEMM accumulators are idle in this phase): S0, S1 (64 each), O0, O1 (48 of 64)
constexpr uint32_t kTcS = 0, kTcO = 128;

// Diagnostics build (CCK_STAGE_REC): the first softmax thread of every CTA adds the cycles it spent in
// each section of an item to row 30 of the stage record (sections: 0 wait for S, 1 S out
// of TMEM, 2 scale + bias + maximum, 3 exchange of the maxima, 4 exponentials and P, 5 hand-over of P,
// 6 wait for the previous O, 7 O out of TMEM and rescale, 8 item prologue, 9 item epilogue; 15: chunks)
#if CCK_STAGE_REC
#define CCK_ATTN_T(k)                                                          \
    do {                                                                       \
        if (threadIdx.x == kWorkWarp0 * 32) {                                  \
            const unsigned long long t_ = clock64();                           \
            atomicAdd(&g_stage_rec[30][k], t_ - at_);                          \
            at_ = t_;                                                          \
        }                                                                      \
    } while (0)
#else
#define CCK_ATTN_T(k) do { } while (0)
#endif

struct TcBars {
    uint64_t q_full[2], q_empty[2];
    uint64_t kv_full[kTcStages], kv_empty[kTcStages];
    uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
};
// per-thread positions, kept across items and phases
static_assert(kTcBarsOff + sizeof(TcBars) <= 1024, "the attention barriers outgrew the control block");
struct TcPipe {
    uint32_t item = 0;  // items started by this role
    uint32_t chunk = 0; // chunks started by this role (all items)
};

__device__ __forceinline__ TcBars* tc_bars() {
    return reinterpret_cast<TcBars*>(smem_base() + kCtlOff + kTcBarsOff);
}
__device__ inline void attn_tc_init() {
    if (threadIdx.x == 0) {
        TcBars* b = tc_bars();
        for (int i = 0; i < 2; i++) {
            mbar_init(&b->q_full[i], 1), mbar_init(&b->q_empty[i], 1);
            mbar_init(&b->s_full[i], 1), mbar_init(&b->o_full[i], 1);
            mbar_init(&b->p_full[i], kWorkWarps * 32), mbar_init(&b->o_free[i], kWorkWarps * 32);
        }
        for (int i = 0; i < kTcStages; i++) {
            mbar_init(&b->kv_full[i], 1), mbar_init(&b->kv_empty[i], 1);
        }
        fence_mbar_init();
    }
}

// 8 f32 columns of this warp's 32 TMEM lanes, without the wait
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
}
// 16 f32 columns of this warp's 32 TMEM lanes, without the wait
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Item it -> (sample, head, block of queries). With barriers around the phase, consecutive items are
// the samples of one (head, block of queries): they share its pair logits. On completion counters
// the items of a sample come together, blocks of queries in order: a sample starts as soon as its
// rows of QKVG are complete, and the rows of TO that a tile of WO reads are complete early.
struct TcItem {
    int s, h, qb;
};
__device__ __forceinline__ TcItem tc_item(int it, int S, int qblocks, bool flow) {
    TcItem i;
    if (flow) {
        i.s = it / (kHeads * qblocks), i.qb = it / kHeads % qblocks, i.h = it % kHeads;
    } else {
        i.s = it % S, i.h = it / S % kHeads, i.qb = it / (S * kHeads);
    }
    return i;
}

// one phase: all items of this CTA
__device__ CCK_PHASE_FN int token_attention_tc(const Launch& L, const Deal d, TcPipe& tp_state, int b) {
    TcPipe tp = tp_state; // in registers while the phase runs: the state itself lives in shared memory
#if CCK_STAGE_REC
    const unsigned long long at0_ = clock64();
#endif
    const KP& p = kp();
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    TcBars* bars = tc_bars();
    const int N = p.N, np = p.np, npb = p.npb, S = p.S;
    const int qblocks = cdiv(N, 128), items = kHeads * qblocks * S, chunks = np / kTcKeys;
    const int warp = warp_id(), lane = lane_id();
    const uint32_t tmem = ctl->tmem_base;
    const bool flow = p.flow;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        const CUtensorMap* mqk = &L.tmap[TM_T_QK];
        const CUtensorMap* mvt = &L.tmap[TM_T_VT];
        const CUtensorMap* mpl = &L.tmap[TM_T_PLG];
        const unsigned int qkvg_done = (unsigned int)(gd_table()[GD_TOK_QKVG].nt * kWorkWarps);
        int ready = -1; // the sample whose rows of QKVG are known to be complete
        for (int it = d.first(); it < items; it += gridDim.x, tp.item++) {
            const TcItem ti = tc_item(it, S, qblocks, flow);
            const int s = ti.s, h = ti.h, qb = ti.qb;
            if (flow && s != ready) {
                // every column tile of QKVG over the sample's rows (q, k, v and the gate), and over the
                // next sample's rows that the last chunk of keys reaches into (masked, but read)
#if CCK_STAGE_REC
                const long long fw0_ = clock64();
#endif
                flow_wait(flow_cnt(p, FC_QKVG), s * N / kBM, (min(s * N + np, S * N) - 1) / kBM, qkvg_done, &ctl->abort);
#if CCK_STAGE_REC
                atomicAdd(&g_stage_rec[28][1], (unsigned long long)(clock64() - fw0_)); // the TMA thread's waits for QKVG
#endif
                ready = s;
            }
            const uint32_t qi = tp.item & 1, qpar = (tp.item >> 1) & 1;
            mbar_wait(&bars->q_empty[qi], qpar ^ 1, &ctl->abort);
            mbar_expect_tx(&bars->q_full[qi], kTcQBytes);
            char* qs = sm + kTcQOff + qi * kTcQBytes;
            tma_load_2d(qs, mqk, h * kHeadD, s * N + qb * 128, &bars->q_full[qi]);
            tma_load_2d(qs + kTcQBytes / 2, mqk, h * kHeadD, s * N + qb * 128 + 64, &bars->q_full[qi]);
            for (int c = 0; c < chunks; c++, tp.chunk++) {
                const uint32_t st = tp.chunk % kTcStages, par = (tp.chunk / kTcStages) & 1;
                mbar_wait(&bars->kv_empty[st], par ^ 1, &ctl->abort);
                mbar_expect_tx(&bars->kv_full[st], kTcStageBytes);
                char* ks = sm + st * kTcStageBytes;
                tma_load_2d(ks, mqk, kTokC + h * kHeadD, s * N + c * kTcKeys, &bars->kv_full[st]);
                tma_load_2d(ks + kTcKBytes, mvt, c * kTcKeys, (s * kHeads + h) * kHeadD, &bars->kv_full[st]);
                tma_load_2d(ks + kTcKBytes + kTcVBytes, mpl, c * kTcKeys, (b * kHeads + h) * npb + qb * 128, &bars->kv_full[st]);
                CCK_STAMP(0, true);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc_s = umma_idesc_bf16(128, kTcKeys), idesc_o = umma_idesc_bf16(128, kHeadD);
        for (int it = d.first(); it < items; it += gridDim.x, tp.item++) {
            const uint32_t qi = tp.item & 1, qpar = (tp.item >> 1) & 1;
            mbar_wait(&bars->q_full[qi], qpar, &ctl->abort);
            tc_fence_after();
            const uint64_t dq = umma_desc_sw128(smem_u32(sm + kTcQOff + qi * kTcQBytes));
            // S of chunk g (global chunk counter) = Q·K_gᵀ; its ring stage and buffers follow from g
            auto issue_qk = [&](uint32_t g) {
                const uint32_t st = g % kTcStages, par = (g / kTcStages) & 1;
                mbar_wait(&bars->kv_full[st], par, &ctl->abort);
                CCK_STAMP(1, true);
                tc_fence_after();
                const uint64_t dk = umma_desc_sw128(smem_u32(sm + st * kTcStageBytes));
#pragma unroll
                for (int kk = 0; kk < kHeadD / 16; kk++) {
                    umma_bf16(tmem + kTcS + (g & 1) * 64, dq + 2 * kk, dk + 2 * kk, idesc_s, kk != 0);
                }
                umma_commit(&bars->s_full[g & 1]);
            };
            issue_qk(tp.chunk);
            for (int c = 0; c < chunks; c++, tp.chunk++) {
                const uint32_t g = tp.chunk, bi = g & 1, bpar = (g >> 1) & 1, st = g % kTcStages;
                if (c + 1 < chunks) {
                    issue_qk(g + 1); // its S buffer was freed when P of chunk g-1 was handed over
                } else {
                    umma_commit(&bars->q_empty[qi]); // every QKᵀ of the item is issued
                }
                mbar_wait(&bars->p_full[bi], bpar, &ctl->abort);     // P of chunk g is in shared memory
                mbar_wait(&bars->o_free[bi], bpar ^ 1, &ctl->abort); // O buffer read out (chunk g-2)
                tc_fence_after();
                const uint64_t dp = umma_desc_sw128(smem_u32(sm + kTcPOff + bi * kTcPBytes));
                const uint64_t dv = umma_desc_sw128(smem_u32(sm + st * kTcStageBytes + kTcKBytes));
#pragma unroll
                for (int kk = 0; kk < kTcKeys / 16; kk++) {
                    umma_bf16(tmem + kTcO + bi * 64, dp + 2 * kk, dv + 2 * kk, idesc_o, kk != 0);
                }
                umma_commit(&bars->o_full[bi]);
                umma_commit(&bars->kv_empty[st]);
                CCK_STAMP(2, false);
            }
        }
    } else if (warp >= kWorkWarp0) {
        // ---- softmax: two threads per query row, each on one half of a chunk's 64 keys and one
        // half of the head's 48 output dims; the halves meet at a named barrier per TMEM lane quarter
        const int q = work_quarter(), hf = work_group(), row_in = q * 32 + lane;
        const uint32_t lane_addr = uint32_t(q * 32) << 16;
        const float scale = kLog2e / sqrtf(float(kHeadD));
        float* xm = reinterpret_cast<float*>(sm + kTcXOff); // [chunk parity][half][row]: chunk maxima
        float* xl = xm + 2 * 2 * 128;                        // [half][row]: row sums
        constexpr int kHalfD = kHeadD / 2;
#if CCK_STAGE_REC
        unsigned long long at_ = clock64();
#endif
        for (int it = d.first(); it < items; it += gridDim.x, tp.item++) {
            const TcItem ti = tc_item(it, S, qblocks, flow);
            const int s = ti.s, h = ti.h, qb = ti.qb;
            float o[kHalfD];
#pragma unroll
            for (int i = 0; i < kHalfD; i++) {
                o[i] = 0.f;
            }
            float m = -INFINITY, l = 0.f, corr_prev = 1.f;
            const int qrow = qb * 128 + row_in;
            const size_t row = size_t(s) * N + min(qrow, N - 1);
            // The row's gate values, fetched now: an L2 round trip that the item's end need not wait for.
            // On completion counters not before the item's Q tile has landed: the TMA thread has then
            // seen the sample's rows of QKVG complete; from L2, where the other CTAs' stores are.
            if (flow) {
                mbar_wait(&bars->q_full[tp.item & 1], (tp.item >> 1) & 1, &ctl->abort);
            }
            uint4 gw[kHalfD / 8];
#pragma unroll
            for (int j = 0; j < kHalfD / 8; j++) {
                gw[j] = __ldcg(reinterpret_cast<const uint4*>(p.buf.qkvg + row * kQKVG + 3 * kTokC + h * kHeadD + kHalfD * hf) + j);
            }
            // O_c of chunk g (this thread's 24 dims), rescaled into the running output
            auto take_o = [&](uint32_t g, float corr) {
                const uint32_t pb = g & 1, ppar = (g >> 1) & 1;
                mbar_wait(&bars->o_full[pb], ppar, &ctl->abort);
                tc_fence_after();
                CCK_ATTN_T(6);
                uint32_t r0[16], r1[8];
                tmem_ld16_issue(tmem + kTcO + pb * 64 + kHalfD * hf + lane_addr, r0);
                tmem_ld8_issue(tmem + kTcO + pb * 64 + kHalfD * hf + 16 + lane_addr, r1);
                tmem_ld_wait(r0);
                tmem_ld_wait(r1);
                tc_fence_before();
                mbar_arrive(&bars->o_free[pb]);
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    o[i] = o[i] * corr + __uint_as_float(r0[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    o[16 + i] = o[16 + i] * corr + __uint_as_float(r1[i]);
                }
                CCK_ATTN_T(7);
            };
            for (int c = 0; c < chunks; c++, tp.chunk++) {
                const uint32_t g = tp.chunk, bi = g & 1, bpar = (g >> 1) & 1, st = g % kTcStages;
                if (c == 0) {
                    CCK_ATTN_T(8);
                }
                // (the chunk's tile of pair logits has landed with K and V: the MMA thread waited for the stage
                // before it issued the Q·Kᵀ whose completion s_full reports)
                mbar_wait(&bars->s_full[bi], bpar, &ctl->abort);
                tc_fence_after();
                CCK_ATTN_T(0);
                uint32_t sr[32];
                tmem_ld32_issue(tmem + kTcS + bi * 64 + 32 * hf + lane_addr, sr);
                // the row's 32 pair logits of this half: 4 swizzled 16-byte pieces of the bias tile
                const char* brow = sm + st * kTcStageBytes + kTcKBytes + kTcVBytes + row_in * 128;
                uint4 bw[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    bw[j] = *reinterpret_cast<const uint4*>(brow + (((4 * hf + j) ^ (row_in & 7)) << 4));
                }
                tmem_ld_wait(sr);
                CCK_ATTN_T(1);
                float sc[32];
                float mxp[4] = {m, m, m, m}; // four chains, so that the maxima do not serialise
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t w[4] = {bw[j].x, bw[j].y, bw[j].z, bw[j].w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int i = 8 * j + 2 * k;
                        sc[i] = fmaf(__uint_as_float(sr[i]), scale, __uint_as_float(w[k] << 16));
                        sc[i + 1] = fmaf(__uint_as_float(sr[i + 1]), scale, __uint_as_float(w[k] & 0xFFFF0000u));
                        mxp[k] = max3(mxp[k], sc[i], sc[i + 1]);
                    }
                }
                float mx = max3(mxp[0], mxp[1], fmaxf(mxp[2], mxp[3]));
                // the row maximum over both halves
                CCK_ATTN_T(2);
                xm[(bi * 2 + hf) * 128 + row_in] = mx;
                asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
                mx = fmaxf(mx, xm[(bi * 2 + (hf ^ 1)) * 128 + row_in]);
                CCK_ATTN_T(3);
                const float corr = ex2_fast(m - mx);
                m = mx;
                float sump[4] = {0.f, 0.f, 0.f, 0.f};
                char* prow = sm + kTcPOff + bi * kTcPBytes + row_in * 128;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float e[8];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        e[k] = ex2_fast(sc[8 * j + k] - mx);
                        sump[k & 3] += e[k];
                    }
                    *reinterpret_cast<uint4*>(prow + (((4 * hf + j) ^ (row_in & 7)) << 4)) =
                        make_uint4(pack_bf2(e[0], e[1]), pack_bf2(e[2], e[3]), pack_bf2(e[4], e[5]), pack_bf2(e[6], e[7]));
                }
                l = l * corr + ((sump[0] + sump[1]) + (sump[2] + sump[3]));
                CCK_ATTN_T(4);
                fence_async_smem(); // P was written by ordinary stores; the tensor core reads it
                tc_fence_before();
                mbar_arrive(&bars->p_full[bi]);
                CCK_ATTN_T(5);
#if CCK_STAGE_REC
                if (threadIdx.x == kWorkWarp0 * 32) {
                    atomicAdd(&g_stage_rec[30][15], 1ull);
                }
#endif
                // the previous chunk's P·V
                if (c > 0) {
                    take_o(g - 1, corr_prev);
                }
                corr_prev = corr;
            }
            take_o(tp.chunk - 1, corr_prev);
            // the row sum over both halves
            xl[hf * 128 + row_in] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
            l += xl[(hf ^ 1) * 128 + row_in];
            if (qrow < N) {
                const float inv = 1.f / l;
                uint4* op = reinterpret_cast<uint4*>(p.buf.to + row * kTokC + h * kHeadD + kHalfD * hf);
#pragma unroll
                for (int j = 0; j < kHalfD / 8; j++) {
                    const uint32_t w[4] = {gw[j].x, gw[j].y, gw[j].z, gw[j].w};
                    uint32_t out[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        out[k] = pack_bf2(o[8 * j + 2 * k] * inv * bf_to_f32(w[k] & 0xFFFFu),
                                          o[8 * j + 2 * k + 1] * inv * bf_to_f32(w[k] >> 16));
                    }
                    op[j] = make_uint4(out[0], out[1], out[2], out[3]);
                }
            }
            if (flow) { // this warp's rows of TO are stored: one arrival at every block of 128 rows that the item's queries touch
                const int lo = s * N + qb * 128, hi = min(lo + 128, (s + 1) * N) - 1;
                flow_signal(flow_cnt(p, FC_TO), lo / kBM, hi / kBM);
            }
            // the partner reads this item's row sum before the next item's may overwrite it
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
            CCK_ATTN_T(9);
            if (threadIdx.x == kWorkWarp0 * 32) {
                CCK_STAMP(4, false);
            }
        }
    }
#if CCK_STAGE_REC
    if (threadIdx.x == kWorkWarp0 * 32) { // row 28: 0 cycles of the first softmax thread in this phase, 1 the TMA thread's waits for QKVG, 2 phases
        atomicAdd(&g_stage_rec[28][0], (unsigned long long)clock64() - at0_);
        atomicAdd(&g_stage_rec[28][2], 1ull);
    }
#endif
    tp_state = tp;
    return items;
}

} // namespace cck

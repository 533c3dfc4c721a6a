// Token attention on the 5th-generation tensor cores: TO = softmax(q·kᵀ/√48 + L_b)·v ⊙ g.
//
// Item = (head, block of 128 queries, sample). A CTA keeps two items in flight, one per track: a
// track is an independent pipeline with its own shared-memory rings, its own TMEM columns and its own
// group of four softmax warps (one thread per query row), so that the bubbles of one item (its
// prologue and epilogue, the waits inside a chunk) are filled by the other item's arithmetic on the
// same SM sub-partitions. Roles:
//   warps 0 and 10, one thread each   TMA of track 0 and of track 1: the Q tile of an item (128 x 64
//                        columns of QKVG of which 48 are used); per chunk of 64 keys the K tile and the
//                        transposed V tile from VT into a 3-deep ring (a chunk's tiles are asked for one
//                        chunk ahead and stay until its P·V is done), and the 128 x 64 tile of pair
//                        logits into a 2-deep ring of its own, released as soon as the softmax threads
//                        have read it
//   warps 1 and 11, one thread each   tcgen05.mma of track 0 and of track 1. One wait per chunk: once
//                        the group's P of chunk g is complete, O += P·V of chunk g (128 x 48, K = 64,
//                        P read from TMEM) and S = Q·Kᵀ of chunk g + 2 (128 x 64, K = 48) into the S
//                        buffer that chunk g has just left go out back to back, so S is always a chunk
//                        ahead of the softmax and nothing waits for two hand-overs in a row
//   8 softmax warps      track = warp group; thread = query row: S out of TMEM, + pair logits, online
//                        base-2 softmax, P (bf16) into the track's P columns of TMEM; finally
//                        O / l · gate -> TO. The gate rows come into a per-warp stage by asynchronous
//                        copies while the chunks run, the output rows replace them there and leave by
//                        one TMA store per warp; the completion counters of TO are raised for an item
//                        when that store has landed, under the next item's first chunk.
// O stays in TMEM for the whole item: P·V accumulates over the chunks. The exponentials of a row are
// taken against a reference value that follows the row's running maximum lazily: it moves only when
// the maximum has grown by more than 2^8 (a warp decides together, since TMEM accesses are
// warp-wide), and then the row's O and sum are rescaled in place before the chunk's P is handed over.
// Until then P may reach 2^8 instead of 1, which changes nothing in bf16 or f32 but the exponent.
// Math as the reference's token attention (src/diffusion/attention.cuh:145-249): logits in base 2,
// P rounded to bf16 before P·V, row sums from the unrounded P.
#pragma once

#include "attention.cuh"

namespace cck {

constexpr int kTcKeys = 64;                       // keys per chunk
constexpr int kTcTracks = 2;                      // items in flight per CTA
constexpr int kTcWarps = kWorkWarps / kTcTracks;  // softmax warps per item
constexpr int kTcRows = kTcWarps * 32;            // query rows per item = softmax threads per track
static_assert(kTcRows == kBM, "one softmax thread per row of a 128-row UMMA");
static_assert(kTcWarps == kAttnItemWarps, "the completion counters of TO count the warps of an item");
constexpr int kTcTmaWarp1 = kAuxWarp0, kTcMmaWarp1 = kAuxWarp0 + 1; // the second track's TMA and MMA threads
constexpr int kTcKvStages = 3, kTcBiasStages = 2;
constexpr float kTcLazy = 8.f; // the exponentials' reference value trails the running maximum by up to 2^8
constexpr int kTcKBytes = kTcKeys * 128;          // 8 KB: 64 keys x 64 columns
constexpr int kTcVBytes = kHeadD * 128;           // 6 KB: 48 head dims x 64 keys
constexpr int kTcKvBytes = kTcKBytes + kTcVBytes; // 14 KB
constexpr int kTcBiasBytes = kTcRows * 128;       // 16 KB: 128 queries x 64 keys
constexpr int kTcQBytes = kTcRows * 128;          // 16 KB
// shared memory of a track: [Q][K|V ring][pair-logit ring][gate / output stage] = 102 KB
constexpr int kTcKvOff = kTcQBytes, kTcBiasOff = kTcKvOff + kTcKvStages * kTcKvBytes;
// Per softmax warp, a stage for its 32 rows of the gate and then of TO, dense rows of 96 bytes: the gate
// comes in by asynchronous copies with the lanes side by side in a row, the thread that owns a row
// replaces it by its row of the output, and one TMA store takes the 32 rows away. (Stores by the
// threads themselves held a warp for some 3000 cycles per item, however the lanes were laid out.)
constexpr int kTcOutPitch = kHeadD * 2, kTcOutPieces = kTcOutPitch / 16, kTcOutWarpBytes = 32 * kTcOutPitch;
constexpr int kTcOutOff = kTcBiasOff + kTcBiasStages * kTcBiasBytes;
constexpr int kTcTrackBytes = kTcOutOff + kTcWarps * kTcOutWarpBytes;
static_assert(kTcTracks * kTcTrackBytes <= kScratchBytes, "the attention buffers live in the scratch area");
static_assert(kTcTrackBytes % 1024 == 0 && kTcKvBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
// TMEM columns of a track (the GEMM accumulators are idle in this phase): S0, S1 by chunk parity (64
// each), P0, P1 by chunk parity (32 each: 64 keys as bf16 pairs), O (48 of 64)
constexpr uint32_t kTcTrackCols = 256, kTcS = 0, kTcP = 128, kTcO = 192;
static_assert(kTcTracks * kTcTrackCols <= kTmemCols, "two tracks share the CTA's TMEM");

struct TcTrackBars {
    uint64_t q_full, q_empty;                             // TMA -> MMA; MMA (every Q·Kᵀ of the item done) -> TMA
    uint64_t kv_full[kTcKvStages], kv_empty[kTcKvStages]; // TMA -> MMA; MMA (P·V of the chunk done) -> TMA
    uint64_t b_full[kTcBiasStages], b_empty[kTcBiasStages]; // TMA -> softmax; softmax (tile read) -> TMA
    uint64_t s_full[2], p_full[2];                        // MMA -> softmax; softmax (P stored, O rescaled) -> MMA
    uint64_t pv_done[2];                                  // MMA (P·V of the chunk done: O is current, for a rescale)
    uint64_t o_full;                                      // MMA (the item's last P·V done) -> softmax
};
// Pipeline positions are counted per track over the whole launch (every role of a track passes the
// same number of items and chunks in a phase), kept here between phases.
struct TcBars {
    TcTrackBars t[kTcTracks];
    uint32_t items[kTcTracks], chunks[kTcTracks];
};
static_assert(kTcBarsOff + sizeof(TcBars) <= kCtlBytes, "the attention barriers outgrew the control block");

__device__ __forceinline__ TcBars* tc_bars() {
    return reinterpret_cast<TcBars*>(smem_base() + kCtlOff + kTcBarsOff);
}
__device__ inline void attn_tc_init() {
    if (threadIdx.x == 0) {
        TcBars* b = tc_bars();
        for (int t = 0; t < kTcTracks; t++) {
            TcTrackBars& tb = b->t[t];
            mbar_init(&tb.q_full, 1), mbar_init(&tb.q_empty, 1);
            for (int i = 0; i < kTcKvStages; i++) {
                mbar_init(&tb.kv_full[i], 1), mbar_init(&tb.kv_empty[i], 1);
            }
            for (int i = 0; i < kTcBiasStages; i++) {
                mbar_init(&tb.b_full[i], 1), mbar_init(&tb.b_empty[i], kTcRows);
            }
            for (int i = 0; i < 2; i++) {
                mbar_init(&tb.s_full[i], 1), mbar_init(&tb.p_full[i], kTcRows), mbar_init(&tb.pv_done[i], 1);
            }
            mbar_init(&tb.o_full, 1);
            b->items[t] = 0, b->chunks[t] = 0;
        }
        fence_mbar_init();
    }
}

// has the phase with this parity completed? Never blocks.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// D[tmem] (+)= A[tmem] · B[smem]ᵀ: A's 128 rows are the TMEM lanes, a 32-bit column holds two
// consecutive k (16 bf16 of k = 8 columns)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
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
// 8 columns of this warp's 32 TMEM lanes from registers (lane l writes TMEM lane base + l)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Item it -> (sample, head, block of queries). With barriers around the phase, consecutive items are
// the samples of one (head, block of queries): they share its pair logits. On completion counters
// the items of a sample come together, blocks of queries in order: a sample starts as soon as its
// rows of QKVG are complete, and the rows of TO that a tile of WO reads are complete early.
struct TcItem {
    int s, h, qb;
};
__device__ __forceinline__ TcItem tc_item(int it, int S, int qblocks, bool flow) {
    // (a division by a number known only at run time costs a chain of some hundred cycles, at the
    // start of every item: the multipliers are prepared once)
    const KP& p = kp();
    TcItem i;
    if (flow) {
        const uint32_t u = uint32_t(it) / kHeads, v = p.tc_div_qblocks ? __umulhi(u, p.tc_div_qblocks) : u;
        i.s = int(v), i.qb = int(u) - int(v) * qblocks, i.h = it % kHeads;
    } else {
        const uint32_t u = p.tc_div_s ? __umulhi(uint32_t(it), p.tc_div_s) : uint32_t(it);
        i.s = it - int(u) * S, i.h = int(u % kHeads), i.qb = int(u / kHeads);
    }
    return i;
}
// The CTA's items of a phase are first, first + grid, ...; track t takes every second one from the
// t-th on. How many that is:
__device__ __forceinline__ int tc_track_items(int first, int items, int t) {
    const int mine = items > first ? (items - first + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    return (mine - t + kTcTracks - 1) / kTcTracks;
}
__device__ __forceinline__ int tc_track_item(int first, int t, int j) {
    return first + (t + kTcTracks * j) * int(gridDim.x);
}
// one phase: all items of this CTA
__device__ CCK_PHASE_FN int token_attention_tc(const Launch& L, const Deal d, int b, unsigned int epoch) {
    const KP& p = kp();
    char* sm = smem_base();
    SmemCtl* ctl = smem_ctl();
    TcBars* bars = tc_bars();
    const int N = p.N, np = p.np, npb = p.npb, S = p.S;
    const int qblocks = cdiv(N, kTcRows), items = kHeads * qblocks * S, chunks = np / kTcKeys;
    const int warp = warp_id(), lane = lane_id(), first = d.first();
    const uint32_t tmem = ctl->tmem_base;
    const bool flow = p.flow;

    if ((warp == 0 || warp == kTcTmaWarp1) && lane == 0) {
        // ---- TMA producer of one track. Issue order: the chunk's pair logits, then K and V of the
        // chunk after it (their slots free up in that order), then, after an item's last chunk, the
        // next item's Q tile (free once every Q·Kᵀ of the item is done).
        const int t = warp != 0;
        const int n = tc_track_items(first, items, t);
        if (n > 0) {
            TcTrackBars& B = bars->t[t];
            char* base = sm + t * kTcTrackBytes;
            const CUtensorMap* mqk = &L.tmap[TM_T_QK];
            const CUtensorMap* mvt = &L.tmap[TM_T_VT];
            const CUtensorMap* mpl = &L.tmap[TM_T_PLG];
            const unsigned int qkvg_done = (epoch + 1) * (unsigned int)(gd_table()[GD_TOK_QKVG].nt * kWorkWarps); // (the counters count on through the launch)
            const uint32_t j0 = bars->items[t], g0 = bars->chunks[t];
            CCK_TRACE_BEGIN(t);
            int ready = -1; // the sample whose rows of QKVG are known to be complete
            auto wait_rows = [&](const TcItem& ti) {
                if (flow && ti.s != ready) {
                    // every column tile of QKVG over the sample's rows (q, k, v and the gate), and over the
                    // next sample's rows that the last chunk of keys reaches into (masked, but read)
                    flow_wait(flow_cnt(p, FC_QKVG), ti.s * N / kBM, (min(ti.s * N + np, S * N) - 1) / kBM, qkvg_done, &ctl->abort);
                    ready = ti.s;
                }
            };
            auto load_q = [&](const TcItem& ti, uint32_t jg) {
                mbar_wait(&B.q_empty, (jg & 1) ^ 1, &ctl->abort);
                mbar_expect_tx(&B.q_full, kTcQBytes);
                tma_load_2d(base, mqk, ti.h * kHeadD, ti.s * N + ti.qb * kTcRows, &B.q_full);
                tma_load_2d(base + kTcQBytes / 2, mqk, ti.h * kHeadD, ti.s * N + ti.qb * kTcRows + 64, &B.q_full);
            };
            auto load_kv = [&](const TcItem& ti, int c, uint32_t g) {
                const uint32_t st = g % kTcKvStages, par = (g / kTcKvStages) & 1;
                mbar_wait(&B.kv_empty[st], par ^ 1, &ctl->abort);
                char* ks = base + kTcKvOff + st * kTcKvBytes;
                mbar_expect_tx(&B.kv_full[st], kTcKvBytes);
                tma_load_2d(ks, mqk, kTokC + ti.h * kHeadD, ti.s * N + c * kTcKeys, &B.kv_full[st]);
                tma_load_2d(ks + kTcKBytes, mvt, c * kTcKeys, (ti.s * kHeads + ti.h) * kHeadD, &B.kv_full[st]);
            };
            auto load_bias = [&](const TcItem& ti, int c, uint32_t g) {
                const uint32_t st = g % kTcBiasStages, par = (g / kTcBiasStages) & 1;
                mbar_wait(&B.b_empty[st], par ^ 1, &ctl->abort);
                mbar_expect_tx(&B.b_full[st], kTcBiasBytes);
                tma_load_2d(base + kTcBiasOff + st * kTcBiasBytes, mpl, c * kTcKeys, (b * kHeads + ti.h) * npb + ti.qb * kTcRows, &B.b_full[st]);
            };
            TcItem cur = tc_item(tc_track_item(first, t, 0), S, qblocks, flow);
            if (t == 1 && p.attn_skew > 0) { // a test's skew between the pipelines: results must not depend on it
                const long long t0 = clock64();
                while (clock64() - t0 < p.attn_skew + 37 * int(blockIdx.x % 64)) {
                }
            }
            wait_rows(cur);
            load_kv(cur, 0, g0);
            load_q(cur, j0);
            CCK_STAMP(0, true);
            uint32_t g = g0;
#pragma unroll 1
            for (int j = 0; j < n; j++) {
#pragma unroll 1
                for (int c = 0; c < chunks; c++, g++) {
                    load_bias(cur, c, g);
                    CCK_TRACE_EV(0x10 + t, g - g0);
                    if (c + 1 < chunks) {
                        load_kv(cur, c + 1, g + 1);
                        CCK_TRACE_EV(0x12 + t, g + 1 - g0);
                    } else if (j + 1 < n) {
                        cur = tc_item(tc_track_item(first, t, j + 1), S, qblocks, flow);
                        wait_rows(cur);
                        load_kv(cur, 0, g + 1);
                        load_q(cur, j0 + j + 1);
                    }
                }
            }
            CCK_TRACE_END();
        }
    } else if ((warp == 1 || warp == kTcMmaWarp1) && lane == 0) {
        // ---- MMA issuer of one track. One wait per chunk: when the group's P of chunk i is complete (and
        // with it everybody has read S of chunk i), O (+)= P·V of chunk i and S of chunk i + 2 go out
        // back to back. Everything an MMA needs is prepared: descriptors differ by constants.
        const int t = warp != 1;
        const int n = tc_track_items(first, items, t), total = n * chunks;
        if (total > 0) {
            TcTrackBars& B = bars->t[t];
            char* base = sm + t * kTcTrackBytes;
            const uint32_t tt = tmem + t * kTcTrackCols;
            const uint32_t idesc_s = umma_idesc_bf16(kTcRows, kTcKeys), idesc_o = umma_idesc_bf16(kTcRows, kHeadD);
            const uint32_t j0 = bars->items[t], g0 = bars->chunks[t];
            const uint64_t dq = umma_desc_sw128(smem_u32(base)), dk0 = umma_desc_sw128(smem_u32(base + kTcKvOff));
            constexpr uint64_t kStageStep = kTcKvBytes >> 4, kVStep = kTcKBytes >> 4; // in the descriptor's address units
            // the next S to issue: chunk number within the phase, its chunk within the item, its item
            int qk_i = 0, qk_c = 0, qk_j = 0;
            uint32_t qk_g = g0;
            // S of the next chunk = Q·Kᵀ. Its S buffer was read by the whole group (the caller has seen the
            // group's P of the chunk two before complete, or the phase has just begun).
            auto issue_qk = [&]() {
                const uint32_t st = qk_g % kTcKvStages;
                if (qk_c == 0) {
                    mbar_wait(&B.q_full, (j0 + uint32_t(qk_j)) & 1, &ctl->abort);
                }
                mbar_wait(&B.kv_full[st], (qk_g / kTcKvStages) & 1, &ctl->abort);
                CCK_STAMP(1, true);
                tc_fence_after();
                const uint64_t dk = dk0 + st * kStageStep;
#pragma unroll
                for (int kk = 0; kk < kHeadD / 16; kk++) {
                    umma_bf16(tt + kTcS + (qk_g & 1) * 64, dq + 2 * kk, dk + 2 * kk, idesc_s, kk != 0);
                }
                umma_commit(&B.s_full[qk_g & 1]);
                qk_i++, qk_g++;
                if (++qk_c == chunks) {
                    umma_commit(&B.q_empty); // every Q·Kᵀ of the item is issued
                    qk_c = 0, qk_j++;
                }
            };
            // S stays two chunks ahead of the softmax. Within the current item the thread waits for what a
            // chunk needs (K lands well ahead); a chunk of the next item goes out ahead only if its Q and K
            // are there already (its sample's rows of QKVG may still be in the making), else when that item starts.
            auto pump = [&](int upto, int item) {
                while (qk_i < upto && qk_i < total) {
                    if (qk_j != item) {
                        const bool ready = mbar_test(&B.kv_full[qk_g % kTcKvStages], (qk_g / kTcKvStages) & 1) &&
                                           (qk_c != 0 || mbar_test(&B.q_full, (j0 + uint32_t(qk_j)) & 1));
                        if (!ready) {
                            break;
                        }
                    }
                    issue_qk();
                }
            };
            tc_fence_after();
            uint32_t g = g0;
            int i = 0;
            CCK_TRACE_BEGIN(2 + t);
#pragma unroll 1
            for (int j = 0; j < n; j++) {
                pump(i + 2, j);
#pragma unroll 1
                for (int c = 0; c < chunks; c++, g++, i++) {
                    const uint32_t bi = g & 1, st = g % kTcKvStages;
                    mbar_wait(&B.p_full[bi], (g >> 1) & 1, &ctl->abort);
                    tc_fence_after();
                    CCK_TRACE_EV(0x20 + t, i);
                    const uint64_t dv = dk0 + st * kStageStep + kVStep;
#pragma unroll
                    for (int kk = 0; kk < kTcKeys / 16; kk++) {
                        umma_bf16_ts(tt + kTcO, tt + kTcP + bi * 32 + 8 * kk, dv + 2 * kk, idesc_o, (c | kk) != 0);
                    }
                    umma_commit(&B.pv_done[bi]);
                    umma_commit(&B.kv_empty[st]);
                    CCK_TRACE_EV(0x22 + t, i);
                    if (c + 1 == chunks) {
                        umma_commit(&B.o_full); // the item's O is complete
                    }
                    CCK_STAMP(2, false);
                    pump(i + 3, j);
                    CCK_TRACE_EV(0x24 + t, i);
                }
            }
            CCK_TRACE_END();
        }
    } else if (warp >= kWorkWarp0 && warp < kAuxWarp0) {
        // ---- softmax: this thread owns one query row of its track's items
        const int t = work_group(), q = work_quarter(), row_in = q * 32 + lane;
        TcTrackBars& B = bars->t[t];
        const char* base = sm + t * kTcTrackBytes;
        char* stage = sm + t * kTcTrackBytes + kTcOutOff + q * kTcOutWarpBytes;
        const uint32_t tt = tmem + t * kTcTrackCols + (uint32_t(q * 32) << 16);
        const float scale = kLog2e / sqrtf(float(kHeadD));
        const float2 scale2 = make_float2(scale, scale);
        const int n = tc_track_items(first, items, t);
        const uint32_t j0 = bars->items[t], g0 = bars->chunks[t];
        uint32_t g = g0;
        // This warp's rows of TO of the item before: one arrival at every block of 128 rows that the
        // item's queries touch, once the TMA store has completed.
        int pend_lo = -1, pend_hi = -1;
        auto publish = [&]() {
            if (lane == 0) {
                bulk_wait_done();
            }
            if (pend_lo >= 0) {
                flow_signal(flow_cnt(p, FC_TO), pend_lo / kBM, pend_hi / kBM);
                pend_lo = -1;
            }
        };
        CCK_TRACE_BEGIN_IF(4 + t, row_in == 0);
#pragma unroll 1
        for (int j = 0; j < n; j++) {
            CCK_TRACE_EV(0x44 + t, j);
            const TcItem ti = tc_item(tc_track_item(first, t, j), S, qblocks, flow);
            const int s = ti.s, h = ti.h, qb = ti.qb;
            const uint32_t jg = j0 + j;
            float m = 0.f, l = 0.f; // the reference value of the row's exponentials, the row sum against it
#pragma unroll 1
            for (int c = 0; c < chunks; c++, g++) {
                const uint32_t bi = g & 1, bpar = (g >> 1) & 1, bst = g % kTcBiasStages;
                CCK_TRACE_EV(0x30 + t, g - g0);
                mbar_wait(&B.s_full[bi], bpar, &ctl->abort);
                tc_fence_after();
                CCK_TRACE_EV(0x32 + t, g - g0);
                if (c == 0) {
                    // The warp's rows of the gate, on their way into its stage while the chunks run. (The
                    // TMA thread saw the sample's rows of QKVG complete before it asked for the item's Q
                    // tile, and S of that Q has been seen; the copies read L2, where the other CTAs' stores are.)
                    if (lane == 0) {
                        bulk_wait_read(); // the previous item's store has read the stage
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < kTcOutPieces; i++) {
                        const int pc = i * 32 + lane, r = pc / kTcOutPieces, o = pc % kTcOutPieces;
                        const size_t grow = size_t(s) * N + min(qb * kTcRows + q * 32 + r, N - 1);
                        cp_async16(stage + r * kTcOutPitch + o * 16, p.buf.qkvg + grow * kQKVG + 3 * kTokC + h * kHeadD + o * 8, true);
                    }
                    cp_async_commit();
                }
                uint32_t s0[32], s1[32]; // the row's scores of the chunk's first and second 32 keys
                tmem_ld32_issue(tt + kTcS + bi * 64, s0);
                tmem_ld32_issue(tt + kTcS + bi * 64 + 32, s1);
                // the row's 64 pair logits: 8 swizzled 16-byte pieces of the tile
                mbar_wait(&B.b_full[bst], (g / kTcBiasStages) & 1, &ctl->abort);
                const char* brow = base + kTcBiasOff + bst * kTcBiasBytes + row_in * 128;
                tmem_ld_wait(s0);
                tmem_ld_wait(s1);
                float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}; // four chains, so that the maxima do not serialise
                // scores in base 2 with the pair logits added, in place; the chunk's maximum
                auto add_bias = [&](uint32_t(&sr)[32], int hf) {
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) {
                        const uint4 bw = *reinterpret_cast<const uint4*>(brow + (((4 * hf + jj) ^ (row_in & 7)) << 4));
                        const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const int i = 8 * jj + 2 * k;
                            const float2 a = __ffma2_rn(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), scale2,
                                                        make_float2(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xFFFF0000u)));
                            sr[i] = __float_as_uint(a.x), sr[i + 1] = __float_as_uint(a.y);
                            mxp[k] = max3(mxp[k], a.x, a.y);
                        }
                    }
                };
                add_bias(s0, 0);
                add_bias(s1, 1);
                // The tile is in registers: its slot may be refilled. The refill is a TMA write (async proxy)
                // over what this thread has just read with ordinary loads: the proxy fence orders the two.
                fence_async_smem();
                mbar_arrive(&B.b_empty[bst]);
                const float mx = max3(mxp[0], mxp[1], fmaxf(mxp[2], mxp[3]));
                CCK_TRACE_EV(0x34 + t, g - g0);
                if (c == 0) {
                    m = mx;
                } else if (__any_sync(0xffffffffu, mx > m + kTcLazy)) {
                    // The reference value moves: the rows of this warp rescale what they have accumulated
                    // (every lane, by its own factor: TMEM accesses are warp-wide). O is current once the
                    // previous chunk's P·V is done, and the next P·V waits for this chunk's P.
                    const float mn = fmaxf(m, mx), f = ex2_fast(m - mn);
                    m = mn, l *= f;
                    mbar_wait(&B.pv_done[bi ^ 1], ((g - 1) >> 1) & 1, &ctl->abort);
                    tc_fence_after();
                    // (16 columns at a time: the chunk's 64 scores are live in registers beside them)
#pragma unroll 1
                    for (int i = 0; i < kHeadD; i += 16) {
                        uint32_t r[16];
                        tmem_ld16_issue(tt + kTcO + i, r);
                        tmem_ld_wait(r);
#pragma unroll
                        for (int k = 0; k < 16; k++) {
                            r[k] = __float_as_uint(__uint_as_float(r[k]) * f);
                        }
                        tmem_st16(tt + kTcO + i, r);
                    }
                }
                // The chunk's P buffer held P of chunk g - 2. That chunk's P·V was issued before this chunk's
                // Q·Kᵀ, by the same thread, and the commit behind s_full covers everything issued before it:
                // having seen S, the buffer is free.
                const float2 neg_m = make_float2(-m, -m);
                float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                // P = 2^(score - reference) as bf16: 16 keys are 8 columns
                auto exp_store = [&](const uint32_t(&sr)[32], int hf) {
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {
                        uint32_t pk[8];
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            const float2 x = __fadd2_rn(make_float2(__uint_as_float(sr[16 * jj + 2 * k]), __uint_as_float(sr[16 * jj + 2 * k + 1])), neg_m);
                            const float2 e = make_float2(ex2_fast(x.x), ex2_fast(x.y));
                            sum2[k & 1] = __fadd2_rn(sum2[k & 1], e);
                            pk[k] = pack_bf2(e.x, e.y);
                        }
                        tmem_st8(tt + kTcP + bi * 32 + 16 * hf + 8 * jj, pk);
                    }
                };
                exp_store(s0, 0);
                exp_store(s1, 1);
                l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&B.p_full[bi]);
                CCK_TRACE_EV(0x38 + t, g - g0);
                if (c == 0 && pend_lo >= 0) {
                    publish();
                }
            }
            cp_async_wait<0>();
            __syncwarp(); // the warp's rows of the gate are in its stage
            CCK_TRACE_EV(0x3a + t, j);
            mbar_wait(&B.o_full, jg & 1, &ctl->abort);
            tc_fence_after();
            CCK_TRACE_EV(0x3c + t, j);
            {
                // own row: O / l times the gate, in place of the gate, 16 columns at a time
                const float inv = 1.f / l;
                uint4* mine = reinterpret_cast<uint4*>(stage + lane * kTcOutPitch);
#pragma unroll
                for (int i = 0; i < kHeadD; i += 16) {
                    uint32_t o[16];
                    tmem_ld16_issue(tt + kTcO + i, o);
                    tmem_ld_wait(o);
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {
                        const uint4 gw = mine[i / 8 + jj];
                        const uint32_t w[4] = {gw.x, gw.y, gw.z, gw.w};
                        uint32_t out[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const float a0 = __uint_as_float(o[8 * jj + 2 * k]), a1 = __uint_as_float(o[8 * jj + 2 * k + 1]);
                            out[k] = pack_bf2(a0 * inv * bf_to_f32(w[k] & 0xFFFFu), a1 * inv * bf_to_f32(w[k] >> 16));
                        }
                        mine[i / 8 + jj] = make_uint4(out[0], out[1], out[2], out[3]);
                    }
                }
                CCK_TRACE_EV(0x40 + t, j);
                tc_fence_before(); // (the next item's first P·V, which overwrites O, follows the group's P of that chunk: after this read)
                // the warp's 32 rows to TO. A sample's last rows may be fewer (the rows after them are the
                // next sample's): those go out row by row.
                const int row0 = qb * kTcRows + q * 32, rows = min(N - row0, 32);
                if (rows == 32) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&L.tmap[TM_T_TO], h * kHeadD, s * N + row0, stage);
                        bulk_commit();
                    }
                } else if (lane < rows) {
                    uint4* dst = reinterpret_cast<uint4*>(p.buf.to + (size_t(s) * N + row0 + lane) * kTokC + h * kHeadD);
#pragma unroll
                    for (int jj = 0; jj < kTcOutPieces; jj++) {
                        dst[jj] = mine[jj];
                    }
                }
            }
            CCK_TRACE_EV(0x42 + t, j);
            if (flow) { // to be published once the store has landed: under the next item's first chunk, or after the last item
                pend_lo = s * N + qb * kTcRows, pend_hi = min(pend_lo + kTcRows, (s + 1) * N) - 1;
            }
            CCK_TRACE_EV(0x3e + t, j);
            if (threadIdx.x == kWorkWarp0 * 32) {
                CCK_STAMP(4, false);
            }
        }
        publish(); // (also: this warp's stores have landed before the phase ends)
        CCK_TRACE_END();
        if (q == 0 && lane == 0) { // one thread of the track
            bars->items[t] = j0 + uint32_t(n), bars->chunks[t] = g;
        }
    }
    return items;
}

} // namespace cck

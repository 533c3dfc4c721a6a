// Attention phases. Both keep a query tile's scores in registers (warp-level m16n8k16 bf16 MMA),
// which fits the atom path's 32 x 128 windows exactly and is the first token-attention path.
//   token: 16 heads x 48, item = (head, 128-query block, sample), online base-2 softmax over
//          64-key chunks staged in shared memory, per-head pair-logit bias from PLG, gate on store
//   atom:  4 heads x 32, item = (32-query subset, sample), 128 keys gathered by Q2K, f32 pair
//          logits read in the input's swizzled tile order, one softmax pass (all keys in registers)
// Reference for the math: src/diffusion/attention.cuh:145-249, :313-434.
#pragma once

#include "rows.cuh"

namespace cck {

// ---- warp MMA fragments (m16n8k16, row.col, bf16 -> f32). With g = lane / 4, t = lane % 4:
//   A: a0 = (g, 2t..2t+1), a1 = (g+8, 2t..), a2 = (g, 2t+8..), a3 = (g+8, 2t+8..)
//   B: b0 = (k 2t..2t+1, n g), b1 = (k 2t+8.., n g)
//   C: c0,c1 = (g, 2t), (g, 2t+1); c2,c3 = (g+8, 2t), (g+8, 2t+1)
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four transposed 8x8 b16 matrices; lane 8m + i supplies the address of row i of matrix m
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(row_ptr)));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool ok) {
    const int bytes = ok ? 16 : 0; // zero-fill when the source row does not exist
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t lds32(const bf16* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}
__device__ __forceinline__ uint32_t ldg32(const bf16* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}
// max / sum over the four lanes that share an accumulator row
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ---- token attention
constexpr int kTokQ = 128;            // queries per item: 16 per warp
constexpr int kTokKeys = 64;          // keys per staged chunk
constexpr int kTokLd = kHeadD + 8;    // smem row pitch (bf16): conflict-free fragment reads
constexpr int kTokStage = 2 * kTokKeys * kTokLd; // K then V, in bf16

__device__ __forceinline__ void stage_tok_chunk(const KP& p, bf16* st, const bf16* rows, int k0) {
    constexpr int kPieces = kHeadD / 8;
    for (int i = threadIdx.x; i < kTokKeys * kPieces; i += kThreads) {
        const int j = i / kPieces, pc = i % kPieces, key = k0 + j;
        const bool ok = key < p.N;
        const bf16* src = rows + size_t(ok ? key : 0) * kQKVG + pc * 8;
        cp_async16(st + j * kTokLd + pc * 8, src + kTokC, ok);
        cp_async16(st + kTokKeys * kTokLd + j * kTokLd + pc * 8, src + 2 * kTokC, ok);
    }
}

__device__ __noinline__ void token_attention_item(const KP& p, int b, int h, int qb, int s) {
    bf16* sm = reinterpret_cast<bf16*>(smem_base());
    const int N = p.N, np = p.np;
    const int g = lane_id() >> 2, t = lane_id() & 3;
    const int q0 = qb * kTokQ + warp_id() * 16;
    const bf16* rows = p.buf.qkvg + size_t(s) * N * kQKVG + h * kHeadD;
    const bf16* plg = p.buf.plg + (size_t(b) * kHeads + h) * p.npb * p.npb;
    const float scale = kLog2e / sqrtf(float(kHeadD));

    // query rows of this lane, clamped inside the sample so that loads stay in bounds; clamped
    // rows are computed and never stored
    const int qa = min(q0 + g, N - 1), qb8 = min(q0 + g + 8, N - 1);
    uint32_t fq[3][4];
#pragma unroll
    for (int kk = 0; kk < 3; kk++) {
        fq[kk][0] = ldg32(rows + size_t(qa) * kQKVG + 16 * kk + 2 * t);
        fq[kk][1] = ldg32(rows + size_t(qb8) * kQKVG + 16 * kk + 2 * t);
        fq[kk][2] = ldg32(rows + size_t(qa) * kQKVG + 16 * kk + 8 + 2 * t);
        fq[kk][3] = ldg32(rows + size_t(qb8) * kQKVG + 16 * kk + 8 + 2 * t);
    }
    float o[6][4];
#pragma unroll
    for (int j = 0; j < 6; j++) {
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const bf16* bias0 = plg + size_t(qa) * p.npb + 2 * t;
    const bf16* bias1 = plg + size_t(qb8) * p.npb + 2 * t;

    const int chunks = np / kTokKeys;
    stage_tok_chunk(p, sm, rows, 0);
    cp_async_commit();
    // the bias words of a chunk are fetched one chunk ahead: their latency hides behind the MMAs
    uint32_t bw0[8], bw1[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        bw0[j] = ldg32(bias0 + 8 * j), bw1[j] = ldg32(bias1 + 8 * j);
    }
#pragma unroll 1
    for (int c = 0; c < chunks; c++) {
        cp_async_wait<0>();
        __syncthreads(); // chunk c landed; every warp is done with the other stage
        if (c + 1 < chunks) {
            stage_tok_chunk(p, sm + ((c + 1) & 1) * kTokStage, rows, (c + 1) * kTokKeys);
        }
        cp_async_commit();
        uint32_t nw0[8], nw1[8];
        const int cn = c + 1 < chunks ? c + 1 : c;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            nw0[j] = ldg32(bias0 + cn * kTokKeys + 8 * j), nw1[j] = ldg32(bias1 + cn * kTokKeys + 8 * j);
        }
        const bf16* ks = sm + (c & 1) * kTokStage;
        const bf16* vs = ks + kTokKeys * kTokLd;
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < 3; kk++) {
                const bf16* kp = ks + (8 * j + g) * kTokLd + 16 * kk + 2 * t;
                mma16816(sc[j], fq[kk], lds32(kp), lds32(kp + 8));
            }
        }
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t b0 = bw0[j], b1 = bw1[j];
            sc[j][0] = sc[j][0] * scale + bf_to_f32(b0 & 0xFFFFu);
            sc[j][1] = sc[j][1] * scale + bf_to_f32(b0 >> 16);
            sc[j][2] = sc[j][2] * scale + bf_to_f32(b1 & 0xFFFFu);
            sc[j][3] = sc[j][3] * scale + bf_to_f32(b1 >> 16);
            mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
        }
        mx0 = quad_max(mx0), mx1 = quad_max(mx1);
        const float corr0 = ex2_fast(m0 - mx0), corr1 = ex2_fast(m1 - mx1);
        m0 = mx0, m1 = mx1;
        l0 *= corr0, l1 *= corr1;
#pragma unroll
        for (int j = 0; j < 6; j++) {
            o[j][0] *= corr0, o[j][1] *= corr0, o[j][2] *= corr1, o[j][3] *= corr1;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sc[j][0] = ex2_fast(sc[j][0] - mx0), sc[j][1] = ex2_fast(sc[j][1] - mx0);
            sc[j][2] = ex2_fast(sc[j][2] - mx1), sc[j][3] = ex2_fast(sc[j][3] - mx1);
            l0 += sc[j][0] + sc[j][1];
            l1 += sc[j][2] + sc[j][3];
        }
        // P (bf16) as the A operand over 16 keys per step; V fragments through transposing loads
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const uint32_t pa[4] = {pack_bf2(sc[2 * kk][0], sc[2 * kk][1]), pack_bf2(sc[2 * kk][2], sc[2 * kk][3]),
                                    pack_bf2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]),
                                    pack_bf2(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
            const int mi = lane_id() >> 3, ri = lane_id() & 7;
#pragma unroll
            for (int j = 0; j < 6; j += 2) {
                uint32_t fv[4];
                ldmatrix_x4_trans(fv, vs + (16 * kk + 8 * (mi & 1) + ri) * kTokLd + 8 * (j + (mi >> 1)));
                mma16816(o[j], pa, fv[0], fv[1]);
                mma16816(o[j + 1], pa, fv[2], fv[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            bw0[j] = nw0[j], bw1[j] = nw1[j];
        }
    }
    __syncthreads(); // the next item restages from the first slot
    l0 = quad_sum(l0), l1 = quad_sum(l1);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < 6; j++) {
        const int col = h * kHeadD + 8 * j + 2 * t;
        if (q0 + g < N) {
            const size_t row = size_t(s) * N + q0 + g;
            const uint32_t gt = ldg32(p.buf.qkvg + row * kQKVG + 3 * kTokC + col);
            *reinterpret_cast<uint32_t*>(p.buf.to + row * kTokC + col) =
                pack_bf2(o[j][0] * inv0 * bf_to_f32(gt & 0xFFFFu), o[j][1] * inv0 * bf_to_f32(gt >> 16));
        }
        if (q0 + g + 8 < N) {
            const size_t row = size_t(s) * N + q0 + g + 8;
            const uint32_t gt = ldg32(p.buf.qkvg + row * kQKVG + 3 * kTokC + col);
            *reinterpret_cast<uint32_t*>(p.buf.to + row * kTokC + col) =
                pack_bf2(o[j][2] * inv1 * bf_to_f32(gt & 0xFFFFu), o[j][3] * inv1 * bf_to_f32(gt >> 16));
        }
    }
}

// TO = softmax(q·kᵀ/√48 + L_b)·v ⊙ g; samples fastest so that co-running items share bias tiles in L2
__device__ void token_attention(const KP& p, Deal& d, int b) {
    const int qblocks = cdiv(p.N, kTokQ), items = kHeads * qblocks * p.S;
    for (int it = d.first(); it < items; it += gridDim.x) {
        token_attention_item(p, b, it / p.S % kHeads, it / (p.S * kHeads), it % p.S);
    }
    d.advance(items);
}

// ---- atom attention
constexpr int kAtomLd = 2 * kAtomC + 8; // smem row pitch (bf16) of a staged [k | v] row

constexpr int kAtomWindow = kSubsetKeys * kAtomLd; // bf16 of one staged window

// the window's [k | v] rows (all heads) of item (u, s): 128 rows x 512 bytes, zero where Q2K is -1
__device__ __forceinline__ void stage_atom_window(const KP& p, bf16* sm, int u, int s) {
    const int* q2k = p.geo.q2k + u * kSubsetKeys;
    for (int i = threadIdx.x; i < kSubsetKeys * 32; i += kThreads) {
        const int j = i >> 5, pc = i & 31, key = q2k[j];
        cp_async16(sm + j * kAtomLd + pc * 8, p.buf.akv + (size_t(s) * p.A + (key < 0 ? 0 : key)) * 2 * kAtomC + pc * 8, key >= 0);
    }
}

// one item from its staged window
__device__ __noinline__ void atom_attention_item(const KP& p, const AtomW& w, int b, int u, int s, const bf16* sm) {
    const int A = p.A, nk = kSubsetKeys;
    const int g = lane_id() >> 2, t = lane_id() & 3;
    const int h = warp_id() & 3, qt = warp_id() >> 2; // head, 16-query half

    const size_t row0 = size_t(s) * A + u * kSubset + qt * 16;
    const bf16* qp = p.buf.aqg + row0 * 2 * kAtomC + h * kAtomHeadD;
    uint32_t fq[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; kk++) {
        fq[kk][0] = ldg32(qp + size_t(g) * 2 * kAtomC + 16 * kk + 2 * t);
        fq[kk][1] = ldg32(qp + size_t(g + 8) * 2 * kAtomC + 16 * kk + 2 * t);
        fq[kk][2] = ldg32(qp + size_t(g) * 2 * kAtomC + 16 * kk + 8 + 2 * t);
        fq[kk][3] = ldg32(qp + size_t(g + 8) * 2 * kAtomC + 16 * kk + 8 + 2 * t);
    }
    const float qm0 = p.geo.qmask[u * kSubset + qt * 16 + g] - 1.f, qm1 = p.geo.qmask[u * kSubset + qt * 16 + g + 8] - 1.f;
    // the pair logits of this (block, subset, head, query tile): nk/16 tiles of 256 floats, each
    // stored as [lane][8 values] in the accumulator order of two adjacent 16x8 tiles
    const float* apl = w.apl + ((((size_t(b) * p.NSb + u) * kAtomHeads + h) * 2 + qt) * (nk / 16)) * 256 + lane_id() * 8;
    const float* kmask = p.geo.kmask + u * nk;
    const float scale = 1.f / sqrtf(float(kAtomHeadD));

    float sc[16][4];
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const bf16* kp = sm + (8 * j + g) * kAtomLd + h * kAtomHeadD + 16 * kk + 2 * t;
            mma16816(sc[j], fq[kk], lds32(kp), lds32(kp + 8));
        }
        const float4 bv = *reinterpret_cast<const float4*>(apl + (j >> 1) * 256 + (j & 1) * 4);
        const float km0 = kmask[8 * j + 2 * t] - 1.f, km1 = kmask[8 * j + 2 * t + 1] - 1.f;
        sc[j][0] = (sc[j][0] * scale + kMaskBias * qm0 * km0 + bv.x) * kLog2e;
        sc[j][1] = (sc[j][1] * scale + kMaskBias * qm0 * km1 + bv.y) * kLog2e;
        sc[j][2] = (sc[j][2] * scale + kMaskBias * qm1 * km0 + bv.z) * kLog2e;
        sc[j][3] = (sc[j][3] * scale + kMaskBias * qm1 * km1 + bv.w) * kLog2e;
        mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
    }
    mx0 = quad_max(mx0), mx1 = quad_max(mx1);
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        sc[j][0] = ex2_fast(sc[j][0] - mx0), sc[j][1] = ex2_fast(sc[j][1] - mx0);
        sc[j][2] = ex2_fast(sc[j][2] - mx1), sc[j][3] = ex2_fast(sc[j][3] - mx1);
        l0 += sc[j][0] + sc[j][1];
        l1 += sc[j][2] + sc[j][3];
    }
    l0 = quad_sum(l0), l1 = quad_sum(l1);
    float o[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    }
    const bf16* vs = sm + kAtomC + h * kAtomHeadD;
    const int mi = lane_id() >> 3, ri = lane_id() & 7;
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
        const uint32_t pa[4] = {pack_bf2(sc[2 * kk][0], sc[2 * kk][1]), pack_bf2(sc[2 * kk][2], sc[2 * kk][3]),
                                pack_bf2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pack_bf2(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            uint32_t fv[4];
            ldmatrix_x4_trans(fv, vs + (16 * kk + 8 * (mi & 1) + ri) * kAtomLd + 8 * (j + (mi >> 1)));
            mma16816(o[j], pa, fv[0], fv[1]);
            mma16816(o[j + 1], pa, fv[2], fv[3]);
        }
    }
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int col = h * kAtomHeadD + 8 * j + 2 * t;
        const size_t ra = row0 + g, rb = row0 + g + 8;
        const uint32_t g0 = ldg32(p.buf.aqg + ra * 2 * kAtomC + kAtomC + col);
        const uint32_t g1 = ldg32(p.buf.aqg + rb * 2 * kAtomC + kAtomC + col);
        *reinterpret_cast<uint32_t*>(p.buf.ao + ra * kAtomC + col) =
            pack_bf2(o[j][0] * inv0 * bf_to_f32(g0 & 0xFFFFu), o[j][1] * inv0 * bf_to_f32(g0 >> 16));
        *reinterpret_cast<uint32_t*>(p.buf.ao + rb * kAtomC + col) =
            pack_bf2(o[j][2] * inv1 * bf_to_f32(g1 & 0xFFFFu), o[j][3] * inv1 * bf_to_f32(g1 >> 16));
    }
}

// AO = softmax(q·kᵀ/√32 + 1e9(QMASK-1)(KMASK-1) + APL)·v ⊙ g over the items (subset, sample)
__device__ void atom_attention(const KP& p, Deal& d, const AtomW& w, int b) {
    const int items = p.NS * p.S;
    bf16* sm = reinterpret_cast<bf16*>(smem_base());
    int it = d.first(), buf = 0;
    if (it < items) {
        stage_atom_window(p, sm, it % p.NS, it / p.NS);
    }
    cp_async_commit();
    // two windows: the next item's rows land while this item computes
    for (; it < items; it += gridDim.x, buf ^= 1) {
        cp_async_wait<0>();
        __syncthreads(); // this window landed; every warp is done with the other one
        const int nx = it + gridDim.x;
        if (nx < items) {
            stage_atom_window(p, sm + (buf ^ 1) * kAtomWindow, nx % p.NS, nx / p.NS);
        }
        cp_async_commit();
        atom_attention_item(p, w, b, it % p.NS, it / p.NS, sm + buf * kAtomWindow);
    }
    cp_async_wait<0>();
    __syncthreads();
    d.advance(items);
}

} // namespace cck

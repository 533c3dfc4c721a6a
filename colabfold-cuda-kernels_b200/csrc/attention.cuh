// Atom attention: 4 heads x 32, item = (32-query subset, sample), 128 keys gathered by Q2K. A
// query tile's scores stay in registers (warp-level m16n8k16 bf16 MMA), which fits the 32 x 128
// windows exactly; f32 pair logits are read in the input's swizzled tile order; one softmax pass
// (all keys in registers). Reference for the math: src/diffusion/attention.cuh:313-434.
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
__device__ CCK_PHASE_FN void atom_attention_item(const KP& p, const AtomW& w, int b, int u, int s, const bf16* sm) {
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
__device__ CCK_PHASE_FN void atom_attention(const KP& p, Deal& d, const AtomW& w, int b) {
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
        if (warp_id() < 2 * kAtomHeads) { // one warp per (head, 16-query half)
            atom_attention_item(p, w, b, it % p.NS, it / p.NS, sm + buf * kAtomWindow);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    d.advance(items);
}

} // namespace cck

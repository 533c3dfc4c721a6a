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
// Work unit = (subset, head, sample), one warp each with its own staging area, no CTA-wide
// synchronisation: the ten warps of a CTA sit at different points of load -> scores -> softmax ->
// P·V, which is what hides the latency of the gathered key rows. Samples run fastest so that the
// units that share a subset's pair logits run at the same time and meet in L2.
constexpr int kAwPitch = kAtomHeadD + 8;                     // bf16 per staged row (80 bytes): conflict-free fragment reads
constexpr int kAwHalf = kSubsetKeys * kAwPitch;              // bf16 of the staged K (or V) rows of one head
constexpr int kAwBytes = 2 * kAwHalf * 2 + kSubsetKeys * 4;  // 20.5 KB per warp: K rows, V rows, the key mask
constexpr int kAwWarps = 10; // warps with a window of their own: what the scratch area holds (the last two warps of the CTA sit this phase out)
static_assert(kAwWarps <= kWarps && kAwWarps * kAwBytes <= kScratchBytes, "the atom windows live in the pipeline and epilogue stages");

// What one half (16 queries) of a unit reads from global memory before its first MMA: the query
// fragments, the gates of its outputs, the query masks and the first eight tiles of pair logits.
// Issued as one batch, ahead of the wait for the staged window.
struct AtomHalf {
    uint32_t fq[2][4];
    uint32_t gt[4][2];
    float qm0, qm1;
    float4 bv[8];
    const float* apl;
    size_t row0;
};
__device__ __forceinline__ void atom_half_load(AtomHalf& a, const KP& p, const AtomW& w, int b, int u, int s, int h, int qt) {
    const int g = lane_id() >> 2, t = lane_id() & 3;
    a.row0 = size_t(s) * p.A + u * kSubset + qt * 16;
    const bf16* qp = p.buf.aqg + a.row0 * 2 * kAtomC + h * kAtomHeadD;
#pragma unroll
    for (int kk = 0; kk < 2; kk++) {
        a.fq[kk][0] = ldg32(qp + size_t(g) * 2 * kAtomC + 16 * kk + 2 * t);
        a.fq[kk][1] = ldg32(qp + size_t(g + 8) * 2 * kAtomC + 16 * kk + 2 * t);
        a.fq[kk][2] = ldg32(qp + size_t(g) * 2 * kAtomC + 16 * kk + 8 + 2 * t);
        a.fq[kk][3] = ldg32(qp + size_t(g + 8) * 2 * kAtomC + 16 * kk + 8 + 2 * t);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int col = h * kAtomHeadD + 8 * j + 2 * t;
        a.gt[j][0] = ldg32(p.buf.aqg + (a.row0 + g) * 2 * kAtomC + kAtomC + col);
        a.gt[j][1] = ldg32(p.buf.aqg + (a.row0 + g + 8) * 2 * kAtomC + kAtomC + col);
    }
    a.qm0 = p.geo.qmask[u * kSubset + qt * 16 + g] - 1.f, a.qm1 = p.geo.qmask[u * kSubset + qt * 16 + g + 8] - 1.f;
    // the pair logits of this (block, subset, head, query tile): 8 tiles of 256 floats, each stored
    // as [lane][8 values] in the accumulator order of two adjacent 16x8 tiles
    a.apl = w.apl + ((((size_t(b) * p.NSb + u) * kAtomHeads + h) * 2 + qt) * (kSubsetKeys / 16)) * 256 + lane_id() * 8;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        a.bv[j] = *reinterpret_cast<const float4*>(a.apl + (j >> 1) * 256 + (j & 1) * 4);
    }
}
// the half against the staged window (K rows, V rows, key mask): one softmax pass, all 128 keys in registers
__device__ __forceinline__ void atom_half_compute(AtomHalf& a, const KP& p, int h, const bf16* sm, const float* kmask) {
    const int g = lane_id() >> 2, t = lane_id() & 3;
    const float scale = 1.f / sqrtf(float(kAtomHeadD));
    float sc[16][4];
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const bf16* kp = sm + (8 * j + g) * kAwPitch + 16 * kk + 2 * t;
            mma16816(sc[j], a.fq[kk], lds32(kp), lds32(kp + 8));
        }
        const float4 bv = a.bv[j & 7];
        if (j < 8) { // the tile eight ahead takes the register just freed
            a.bv[j] = *reinterpret_cast<const float4*>(a.apl + ((j + 8) >> 1) * 256 + (j & 1) * 4);
        }
        const float2 km = *reinterpret_cast<const float2*>(kmask + 8 * j + 2 * t);
        const float km0 = km.x - 1.f, km1 = km.y - 1.f;
        sc[j][0] = (sc[j][0] * scale + kMaskBias * a.qm0 * km0 + bv.x) * kLog2e;
        sc[j][1] = (sc[j][1] * scale + kMaskBias * a.qm0 * km1 + bv.y) * kLog2e;
        sc[j][2] = (sc[j][2] * scale + kMaskBias * a.qm1 * km0 + bv.z) * kLog2e;
        sc[j][3] = (sc[j][3] * scale + kMaskBias * a.qm1 * km1 + bv.w) * kLog2e;
        mx0 = max3(mx0, sc[j][0], sc[j][1]);
        mx1 = max3(mx1, sc[j][2], sc[j][3]);
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
    const bf16* vs = sm + kAwHalf;
    const int mi = lane_id() >> 3, ri = lane_id() & 7;
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
        const uint32_t pa[4] = {pack_bf2(sc[2 * kk][0], sc[2 * kk][1]), pack_bf2(sc[2 * kk][2], sc[2 * kk][3]),
                                pack_bf2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pack_bf2(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            uint32_t fv[4];
            ldmatrix_x4_trans(fv, vs + (16 * kk + 8 * (mi & 1) + ri) * kAwPitch + 8 * (j + (mi >> 1)));
            mma16816(o[j], pa, fv[0], fv[1]);
            mma16816(o[j + 1], pa, fv[2], fv[3]);
        }
    }
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int col = h * kAtomHeadD + 8 * j + 2 * t;
        const size_t ra = a.row0 + g, rb = a.row0 + g + 8;
        *reinterpret_cast<uint32_t*>(p.buf.ao + ra * kAtomC + col) =
            pack_bf2(o[j][0] * inv0 * bf_to_f32(a.gt[j][0] & 0xFFFFu), o[j][1] * inv0 * bf_to_f32(a.gt[j][0] >> 16));
        *reinterpret_cast<uint32_t*>(p.buf.ao + rb * kAtomC + col) =
            pack_bf2(o[j][2] * inv1 * bf_to_f32(a.gt[j][1] & 0xFFFFu), o[j][3] * inv1 * bf_to_f32(a.gt[j][1] >> 16));
    }
}

// AO = softmax(q·kᵀ/√32 + 1e9(QMASK-1)(KMASK-1) + APL)·v ⊙ g (reference: src/diffusion/attention.cuh:313-434)
__device__ CCK_HOT_FN void atom_attention(const KP& p, Deal& d, const AtomW& w, int b) {
    const int units = p.NS * kAtomHeads * p.S;
    bf16* sm = reinterpret_cast<bf16*>(smem_base() + warp_id() * kAwBytes);
    const int lane = lane_id();
    for (int un = d.first() * kAwWarps + warp_id(); un < units && warp_id() < kAwWarps; un += gridDim.x * kAwWarps) {
        const int s = un % p.S, h = un / p.S % kAtomHeads, u = un / (p.S * kAtomHeads);
        __syncwarp(); // every lane is done with the previous window
        // the head's slice of the window's [k | v] rows: 128 rows x (64 + 64) bytes, zero where Q2K is -1.
        // Four lanes copy one 64-byte slice, so an instruction touches 8 lines rather than 32.
        const int* q2k = p.geo.q2k + u * kSubsetKeys;
        int keys[kSubsetKeys / 32];
#pragma unroll
        for (int i = 0; i < kSubsetKeys / 32; i++) {
            keys[i] = q2k[lane + 32 * i];
        }
        const int pc = lane & 3;
#pragma unroll
        for (int i = 0; i < kSubsetKeys / 8; i++) {
            const int j = 8 * i + (lane >> 2);
            const int key = __shfl_sync(0xffffffffu, keys[i / 4], j & 31);
            const bf16* src = p.buf.akv + (size_t(s) * p.A + (key < 0 ? 0 : key)) * 2 * kAtomC + h * kAtomHeadD + pc * 8;
            cp_async16(sm + j * kAwPitch + pc * 8, src, key >= 0);
            cp_async16(sm + kAwHalf + j * kAwPitch + pc * 8, src + kAtomC, key >= 0);
        }
        float* kmask = reinterpret_cast<float*>(sm + 2 * kAwHalf);
        cp_async16(kmask + 4 * lane, p.geo.kmask + u * kSubsetKeys + 4 * lane, true);
        cp_async_commit();
        AtomHalf a;
        atom_half_load(a, p, w, b, u, s, h, 0); // under way while the window lands
        cp_async_wait<0>();
        __syncwarp();
        atom_half_compute(a, p, h, sm, kmask);
        atom_half_load(a, p, w, b, u, s, h, 1);
        atom_half_compute(a, p, h, sm, kmask);
    }
    d.advance(cdiv(units, kAwWarps));
}

} // namespace cck

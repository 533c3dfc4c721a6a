// Row phases: one warp per row, 128-bit accesses, warp-shuffle reductions. LayerNorm is two-pass
// in f32. These are the HBM/L2-bound pieces between the GEMMs: conditioning rows, token adaLN,
// atom adaLN inputs, the atom/token glue.
// Reference for the math: src/diffusion/rows.cuh:105-311, src/diffusion/atom_mlp.cuh:339-364,
// :492-517, :559-612, src/diffusion/gemm.cuh:231-256.
#pragma once

#include "gemm.cuh"

namespace cck {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

// a row of 128·NV floats: lane l holds columns 4l + 128j
template <int NV> struct RowV {
    float4 v[NV];
};
// the same from L2: for rows that other CTAs have just written, read after a completion counter
template <int NV> __device__ __forceinline__ RowV<NV> load_f32_cg(const float* p) {
    RowV<NV> r;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        r.v[j] = __ldcg(reinterpret_cast<const float4*>(p + 4 * lane_id() + 128 * j));
    }
    return r;
}
template <int NV> __device__ __forceinline__ RowV<NV> load_f32(const float* p) {
    RowV<NV> r;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        r.v[j] = *reinterpret_cast<const float4*>(p + 4 * lane_id() + 128 * j);
    }
    return r;
}
__device__ __forceinline__ float4 bf4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(bf_to_f32(u.x & 0xFFFFu), bf_to_f32(u.x >> 16), bf_to_f32(u.y & 0xFFFFu), bf_to_f32(u.y >> 16));
}
template <int NV> __device__ __forceinline__ void store_f32(float* p, const RowV<NV>& r) {
#pragma unroll
    for (int j = 0; j < NV; j++) {
        *reinterpret_cast<float4*>(p + 4 * lane_id() + 128 * j) = r.v[j];
    }
}
__device__ __forceinline__ void store_bf4(bf16* p, float4 x) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf2(x.x, x.y), pack_bf2(x.z, x.w));
}
template <int NV> __device__ __forceinline__ void store_bf(bf16* p, const RowV<NV>& r) {
#pragma unroll
    for (int j = 0; j < NV; j++) {
        store_bf4(p + 4 * lane_id() + 128 * j, r.v[j]);
    }
}
// two-pass LayerNorm without affine, in place
template <int NV> __device__ __forceinline__ void layernorm(RowV<NV>& r, float eps) {
    constexpr float n = 128.f * NV;
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        s += r.v[j].x + r.v[j].y + r.v[j].z + r.v[j].w;
    }
    const float mean = warp_sum(s) / n;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        float4& x = r.v[j];
        x.x -= mean, x.y -= mean, x.z -= mean, x.w -= mean;
        q += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    const float rstd = 1.f / sqrtf(warp_sum(q) / n + eps);
#pragma unroll
    for (int j = 0; j < NV; j++) {
        float4& x = r.v[j];
        x.x *= rstd, x.y *= rstd, x.z *= rstd, x.w *= rstd;
    }
}
__device__ __forceinline__ float4 fma4(float4 x, float4 s, float4 o) {
    return make_float4(x.x * s.x + o.x, x.y * s.y + o.y, x.z * s.z + o.z, x.w * s.w + o.w);
}

// rows of a phase: kWarps per CTA item, continuing the phase's rotation
__device__ __forceinline__ int row_first(const Deal& d) {
    return d.first() * kWarps + warp_id();
}
__device__ __forceinline__ int row_step() {
    return gridDim.x * kWarps;
}
__device__ __forceinline__ void rows_done(Deal& d, int rows) {
    d.advance(cdiv(rows, kWarps));
}

// ---- conditioning

// ntv = LN_affine(cos(2π(¼ ln(t/σd)·w + b))) @ WN on one CTA (reference: src/diffusion/rows.cuh:168-200)
__device__ CCK_PHASE_FN void noise_vector(const KP& p, Deal& d, float t) {
    if (d.first() == 0) {
        float* e = reinterpret_cast<float*>(smem_base());
        float* red = e + kFourier;
        const float lt = 0.25f * logf(t / kSigmaData);
        const int k = threadIdx.x; // one thread per Fourier feature; the warps past them add zeros
        const bool on = k < kFourier;
        const float x = on ? cosf(2.f * 3.14159265358979323846f * (lt * p.tw.fourier_w[k] + p.tw.fourier_b[k])) : 0.f;
        float s = warp_sum(x);
        if (lane_id() == 0) {
            red[warp_id()] = s;
        }
        __syncthreads();
        s = 0.f;
        for (int w = 0; w < kWarps; w++) {
            s += red[w];
        }
        const float mean = s / kFourier;
        __syncthreads();
        float q = warp_sum(on ? (x - mean) * (x - mean) : 0.f);
        if (lane_id() == 0) {
            red[warp_id()] = q;
        }
        __syncthreads();
        q = 0.f;
        for (int w = 0; w < kWarps; w++) {
            q += red[w];
        }
        const float rstd = 1.f / sqrtf(q / kFourier + kLnEps);
        if (on) {
            e[k] = (x - mean) * rstd * p.tw.noise_ln[k] + p.tw.noise_lno[k];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < p.cs; c += kThreads) {
            float acc = 0.f;
            for (int j = 0; j < kFourier; j++) {
                acc += e[j] * p.tw.wn[j * p.cs + c];
            }
            p.buf.ntv[c] = acc;
        }
        __syncthreads();
    }
    d.advance(1);
}
static_assert(kThreads >= kFourier, "noise_vector maps one thread to one Fourier feature");

// SCT = bf16(LN(sc)·S + O); the first call also forms sc = SC_BASE + ntv
// (reference: src/diffusion/rows.cuh:202-222). cs = 384.
__device__ CCK_PHASE_FN void sc_layernorm(const KP& p, Deal& d, int i, bool first) {
    for (int n = row_first(d); n < p.N; n += row_step()) {
        RowV<3> x;
        if (first) {
            x = load_f32<3>(p.tw.sc_base + size_t(n) * p.cs);
            const RowV<3> nv = load_f32<3>(p.buf.ntv);
#pragma unroll
            for (int j = 0; j < 3; j++) {
                x.v[j].x += nv.v[j].x, x.v[j].y += nv.v[j].y, x.v[j].z += nv.v[j].z, x.v[j].w += nv.v[j].w;
            }
            store_f32<3>(p.buf.sc + size_t(n) * p.cs, x);
        } else {
            x = load_f32<3>(p.buf.sc + size_t(n) * p.cs);
        }
        layernorm<3>(x, kLnEps);
        const RowV<3> s = load_f32<3>(p.tw.st_s[i]), o = load_f32<3>(p.tw.st_o[i]);
#pragma unroll
        for (int j = 0; j < 3; j++) {
            x.v[j] = fma4(x.v[j], s.v[j], o.v[j]);
        }
        store_bf<3>(p.buf.sct + size_t(n) * p.cs, x);
    }
    rows_done(d, p.N);
}
// SCBF = bf16(sc), SCLN0 = bf16(LN(sc)); SCFINAL: sc goes through an affine LayerNorm first
// (reference: src/diffusion/rows.cuh:224-238)
__device__ CCK_PHASE_FN void sc_prep(const KP& p, Deal& d) {
    for (int n = row_first(d); n < p.N; n += row_step()) {
        RowV<3> x = load_f32<3>(p.buf.sc + size_t(n) * p.cs);
        if (p.flags & F_SCFINAL) {
            layernorm<3>(x, kLnEps);
            const RowV<3> s = load_f32<3>(p.tw.scf), o = load_f32<3>(p.tw.scf + p.cs);
#pragma unroll
            for (int j = 0; j < 3; j++) {
                x.v[j] = fma4(x.v[j], s.v[j], o.v[j]);
            }
        }
        store_bf<3>(p.buf.scbf + size_t(n) * p.cs, x);
        layernorm<3>(x, kLnEps);
        store_bf<3>(p.buf.scln0 + size_t(n) * p.cs, x);
    }
    rows_done(d, p.N);
}

// ---- token rows

__device__ __forceinline__ const bf16* tok_mods(const KP& p, int b, int slot) {
    return p.buf.mods + (size_t(b) * kTokModSlots + slot) * p.N * kTokC;
}
// TX = bf16(LN(act)·mods[slot] + mods[slot+1]) (reference: src/diffusion/rows.cuh:270-285).
// A warp keeps two rows in flight: all loads of both rows are issued before the first reduction.
#ifndef CCK_ADALN_ROWS
#define CCK_ADALN_ROWS 1
#endif
struct AdaRow {
    RowV<6> x;
    uint2 s[6], o[6];
};
// the row's modulations (known since the conditioning ran: nothing to wait for)
__device__ __forceinline__ void adaln_load_mods(AdaRow& a, const KP& p, const bf16* ms, const bf16* mo, int r) {
    const size_t mrow = size_t(r % p.N) * kTokC + 4 * lane_id();
#pragma unroll
    for (int j = 0; j < 6; j++) {
        a.s[j] = *reinterpret_cast<const uint2*>(ms + mrow + 128 * j);
        a.o[j] = *reinterpret_cast<const uint2*>(mo + mrow + 128 * j);
    }
}
__device__ __forceinline__ void adaln_load(AdaRow& a, const KP& p, const bf16* ms, const bf16* mo, int r) {
    a.x = load_f32_cg<6>(p.buf.act + size_t(r) * kTokC);
    adaln_load_mods(a, p, ms, mo, r);
}
__device__ __forceinline__ float4 bf4u(uint2 u) {
    return make_float4(bf_to_f32(u.x & 0xFFFFu), bf_to_f32(u.x >> 16), bf_to_f32(u.y & 0xFFFFu), bf_to_f32(u.y >> 16));
}
__device__ __forceinline__ void adaln_finish(AdaRow& a, const KP& p, int r) {
    layernorm<6>(a.x, p.ln_eps);
#pragma unroll
    for (int j = 0; j < 6; j++) {
        keep_packed(a.s[j]), keep_packed(a.o[j]);
        a.x.v[j] = fma4(a.x.v[j], bf4u(a.s[j]), bf4u(a.o[j]));
    }
    store_bf<6>(p.buf.tx + size_t(r) * kTokC, a.x);
}
// PARALLEL: TX from the attention's modulations and TX2 from the transition's, one LayerNorm
// (reference: src/diffusion/rows.cuh:270-283)
__device__ CCK_PHASE_FN void token_adaln2(const KP& p, Deal& d, int b) {
    const int rows = p.S * p.N;
    const bf16* m = tok_mods(p, b, TM_ATTN_SCALE);
    const bf16* m2 = tok_mods(p, b, TM_TRANS_SCALE);
    const size_t off = size_t(p.N) * kTokC; // the offset row follows the scale row
    for (int r = row_first(d); r < rows; r += row_step()) {
        RowV<6> x = load_f32<6>(p.buf.act + size_t(r) * kTokC);
        layernorm<6>(x, p.ln_eps);
        const size_t mrow = size_t(r % p.N) * kTokC + 4 * lane_id();
        RowV<6> y, y2;
#pragma unroll
        for (int j = 0; j < 6; j++) {
            y.v[j] = fma4(x.v[j], bf4(m + mrow + 128 * j), bf4(m + off + mrow + 128 * j));
            y2.v[j] = fma4(x.v[j], bf4(m2 + mrow + 128 * j), bf4(m2 + off + mrow + 128 * j));
        }
        store_bf<6>(p.buf.tx + size_t(r) * kTokC, y);
        store_bf<6>(p.buf.tx2 + size_t(r) * kTokC, y2);
    }
    rows_done(d, rows);
}
// Token rows under the completion counters: every CTA takes one contiguous run of rows, so that it
// depends on one or two blocks of 128 rows, and a warp starts a row when the tiles of the GEMM that
// wrote ACT over the row's block are complete (cnt counts on through the launch: target is the
// count after the GEMM of the current token block). Returns false when the wait gave up.
struct FlowRows {
    int r0, r1, ok;
    const unsigned int* cnt;
    unsigned int target;
};
__device__ __forceinline__ FlowRows flow_rows(const KP& p, int rows, int which, unsigned int gemms_done) {
    FlowRows f;
    const int per = cdiv(rows, int(gridDim.x));
    f.r0 = min(rows, int(blockIdx.x) * per) + warp_id(), f.r1 = min(rows, (int(blockIdx.x) + 1) * per), f.ok = -1;
    f.cnt = flow_cnt(p, which);
    f.target = gemms_done * (unsigned int)(gd_table()[which == FC_ACT1 ? GD_TOK_WO : GD_TOK_W2].nt * kWorkWarps);
    return f;
}
__device__ __forceinline__ void flow_row_wait(FlowRows& f, int r) {
    const int rb = r / kBM;
    if (rb != f.ok) {
        if (lane_id() == 0) {
            flow_wait(f.cnt, rb, rb, f.target, &smem_ctl()->abort);
        }
        __syncwarp();
        f.ok = rb;
    }
}
__device__ CCK_HOT_FN void token_adaln(const KP& p, Deal& d, int b, int slot, unsigned int epoch) {
    const int rows = p.S * p.N, step = row_step();
    const bf16* ms = tok_mods(p, b, slot);
    const bf16* mo = tok_mods(p, b, slot + 1);
    if (p.flow) {
        // the attention's input follows W2 of the block before, the transition's input WO of this block
        FlowRows f = flow_rows(p, rows, slot == TM_ATTN_SCALE ? FC_ACT2 : FC_ACT1, epoch + (slot != TM_ATTN_SCALE));
        unsigned int* tx_done = flow_cnt(p, FC_TX);
        for (int r = f.r0; r < f.r1; r += kWarps) {
            AdaRow a0;
            adaln_load_mods(a0, p, ms, mo, r); // (nothing to wait for: they travel while the counter is awaited)
            flow_row_wait(f, r);
            a0.x = load_f32_cg<6>(p.buf.act + size_t(r) * kTokC);
            adaln_finish(a0, p, r);
            if (slot != TM_ATTN_SCALE) { // W1's tiles over the row's block of 128 wait for its rows
                flow_signal(tx_done, r / kBM, r / kBM);
            }
        }
        return;
    }
#if CCK_ADALN_ROWS == 1
    for (int r = row_first(d); r < rows; r += step) {
        AdaRow a0;
        adaln_load(a0, p, ms, mo, r);
        adaln_finish(a0, p, r);
    }
#else
    for (int r = row_first(d); r < rows; r += 2 * step) {
        AdaRow a0, a1;
        const bool two = r + step < rows;
        adaln_load(a0, p, ms, mo, r);
        if (two) {
            adaln_load(a1, p, ms, mo, r + step);
        }
        adaln_finish(a0, p, r);
        if (two) {
            adaln_finish(a1, p, r + step);
        }
    }
#endif
    rows_done(d, rows);
}
// QKNORM: LayerNorm of q and of k over their 768 flattened channels with the block's scale and
// offset rows, in place on the bf16 rows of QKVG (reference: src/diffusion/rows.cuh:287-300)
__device__ CCK_PHASE_FN void token_qknorm(const KP& p, Deal& d, int b) {
    const int rows = p.S * p.N;
    for (int r = row_first(d); r < 2 * rows; r += row_step()) {
        const bool is_k = r >= rows;
        bf16* q = p.buf.qkvg + size_t(r - (is_k ? rows : 0)) * kQKVG + (is_k ? kTokC : 0);
        const float* qkn = p.tw.tqkn + (size_t(b) * kQkNormRows + (is_k ? QKN_K_SCALE : QKN_Q_SCALE)) * kTokC;
        RowV<6> x;
#pragma unroll
        for (int j = 0; j < 6; j++) {
            x.v[j] = bf4(q + 4 * lane_id() + 128 * j);
        }
        layernorm<6>(x, kLnEps);
        const RowV<6> s = load_f32<6>(qkn), o = load_f32<6>(qkn + kTokC);
#pragma unroll
        for (int j = 0; j < 6; j++) {
            x.v[j] = fma4(x.v[j], s.v[j], o.v[j]);
        }
        store_bf<6>(q, x);
    }
    rows_done(d, 2 * rows);
}
// TX = bf16(LN(act)) (reference: src/diffusion/rows.cuh:302-311)
__device__ CCK_PHASE_FN void token_final_ln(const KP& p, Deal& d, unsigned int epoch) {
    const int rows = p.S * p.N;
    if (p.flow) { // after W2 of the last token block
        FlowRows f = flow_rows(p, rows, FC_ACT2, epoch);
        for (int r = f.r0; r < f.r1; r += kWarps) {
            flow_row_wait(f, r);
            RowV<6> x = load_f32_cg<6>(p.buf.act + size_t(r) * kTokC);
            layernorm<6>(x, kLnEps);
            store_bf<6>(p.buf.tx + size_t(r) * kTokC, x);
        }
        return;
    }
    for (int r = row_first(d); r < rows; r += row_step()) {
        RowV<6> x = load_f32<6>(p.buf.act + size_t(r) * kTokC);
        layernorm<6>(x, kLnEps);
        store_bf<6>(p.buf.tx + size_t(r) * kTokC, x);
    }
    rows_done(d, rows);
}
// act[s,n] = Σ_j TAM[n,j]·AGT[s, Q2TA[n,j]] / max(Σ_j TAM, 1e-10) + se[n], AGT = relu(abf @ WAGGRᵀ)
// per atom row; the slots are summed in order j = 0..23 as the reference's staged epilogue does
// (src/diffusion/gemm.cuh:231-256)
__device__ CCK_PHASE_FN void aggr_gather(const KP& p, Deal& d) {
    const int rows = p.S * p.N;
    for (int r = row_first(d); r < rows; r += row_step()) {
        const int s = r / p.N, n = r % p.N;
        RowV<6> sum;
#pragma unroll
        for (int j = 0; j < 6; j++) {
            sum.v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float wsum = 0.f;
        for (int j = 0; j < kSlots; j++) {
            const float w = p.geo.tam[n * kSlots + j];
            const int a = p.geo.q2ta[n * kSlots + j];
            wsum += w;
            if (a >= 0) {
                const RowV<6> v = load_f32<6>(p.buf.agt + (size_t(s) * p.A + a) * kTokC);
#pragma unroll
                for (int k = 0; k < 6; k++) {
                    sum.v[k].x += w * v.v[k].x, sum.v[k].y += w * v.v[k].y;
                    sum.v[k].z += w * v.v[k].z, sum.v[k].w += w * v.v[k].w;
                }
            }
        }
        const float inv = 1.f / fmaxf(wsum, 1e-10f);
        const RowV<6> se = load_f32<6>(p.buf.se + size_t(n) * kTokC);
#pragma unroll
        for (int k = 0; k < 6; k++) {
            sum.v[k] = make_float4(sum.v[k].x * inv + se.v[k].x, sum.v[k].y * inv + se.v[k].y,
                                   sum.v[k].z * inv + se.v[k].z, sum.v[k].w * inv + se.v[k].w);
        }
        store_f32<6>(p.buf.act + size_t(r) * kTokC, sum);
    }
    rows_done(d, rows);
}

// ---- atom rows (128 wide: one float4 per lane)

__device__ __forceinline__ const float* atom_mods(const KP& p, const AtomW& w, int b, int a) {
    return w.amods + (size_t(b) * p.NSb * kSubset + a) * kAtomModSlots * kAtomC;
}
__device__ __forceinline__ float4 ld4(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}

// ---- atom rows, four rows per warp: a 128-wide row is only 512 bytes, so eight lanes take one row
// (lane l: row l / 8 of the group, columns 4(l % 8) + 32j, j < 4) and a warp instruction covers four
// rows. Per-row reductions run over the eight lanes of the row.
__device__ __forceinline__ float oct_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v + __shfl_xor_sync(0xffffffffu, v, 4);
}
struct Oct {
    float4 v[4];
};
__device__ __forceinline__ int oct_col() {
    return 4 * (lane_id() & 7);
}
__device__ __forceinline__ Oct oct_load(const float* row) {
    Oct o;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o.v[j] = ld4(row + oct_col() + 32 * j);
    }
    return o;
}
__device__ __forceinline__ void oct_layernorm(Oct& x, float eps) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        s += x.v[j].x + x.v[j].y + x.v[j].z + x.v[j].w;
    }
    const float mean = oct_sum(s) / kAtomC;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float4& v = x.v[j];
        v.x -= mean, v.y -= mean, v.z -= mean, v.w -= mean;
        q += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float rstd = 1.f / sqrtf(oct_sum(q) / kAtomC + eps);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float4& v = x.v[j];
        v.x *= rstd, v.y *= rstd, v.z *= rstd, v.w *= rstd;
    }
}
// rows of a range [first, end) go four to a warp step: this lane's row of step i
__device__ __forceinline__ int oct_row(int first, int i) {
    return first + 4 * (warp_id() + kWarps * i) + (lane_id() >> 3);
}
__device__ __forceinline__ int oct_steps(int first, int end) {
    return cdiv(end - first, 4 * kWarps);
}

// AXQ = bf16(LN(qa)·am0 + am1), AXK = bf16(LN(qa)·am2 + am3): the inputs of the q|g and k|v
// projections (reference: src/diffusion/atom_mlp.cuh:339-364), rows [first, end) by this CTA
__device__ __forceinline__ void atom_ln_qk_rows(const KP& p, const AtomW& w, int b, int first, int end) {
    for (int i = 0; i < oct_steps(first, end); i++) {
        const int r = min(oct_row(first, i), end - 1); // a lane past the end redoes the last row
        const float* am = atom_mods(p, w, b, r % p.A);
        Oct x = oct_load(p.buf.qa + size_t(r) * kAtomC);
        const Oct qs = oct_load(am + AM_Q_SCALE * kAtomC), qb = oct_load(am + AM_Q_BIAS * kAtomC);
        const Oct ks = oct_load(am + AM_K_SCALE * kAtomC), kb = oct_load(am + AM_K_BIAS * kAtomC);
        oct_layernorm(x, p.ln_eps);
        Oct xk = x;
        if (p.flags & F_CHAIN_K) { // the keys' input is normalised from bf16(xq) (reference: src/diffusion/atom_mlp.cuh:349-358)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 q = fma4(x.v[j], qs.v[j], qb.v[j]);
                xk.v[j] = make_float4(round_bf(q.x), round_bf(q.y), round_bf(q.z), round_bf(q.w));
            }
            oct_layernorm(xk, p.ln_eps);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = oct_col() + 32 * j;
            store_bf4(p.buf.axq + size_t(r) * kAtomC + c, fma4(x.v[j], qs.v[j], qb.v[j]));
            store_bf4(p.buf.axk + size_t(r) * kAtomC + c, fma4(xk.v[j], ks.v[j], kb.v[j]));
        }
    }
}
// AXHL = [hi | lo] of x = LN(qa)·am4 + am5 with hi = bf16(x), lo = bf16(x - hi): the transition
// input carried to ~16 mantissa bits (reference: src/diffusion/atom_mlp.cuh:510-517,
// src/diffusion/frag.cuh:396-406)
__device__ __forceinline__ void atom_ln_t_rows(const KP& p, const AtomW& w, int b, int first, int end) {
    for (int i = 0; i < oct_steps(first, end); i++) {
        const int r = min(oct_row(first, i), end - 1);
        const float* am = atom_mods(p, w, b, r % p.A);
        Oct x = oct_load(p.buf.qa + size_t(r) * kAtomC);
        const Oct ts = oct_load(am + AM_T_SCALE * kAtomC), tb = oct_load(am + AM_T_BIAS * kAtomC);
        oct_layernorm(x, p.ln_eps);
        bf16* o = p.buf.axhl + size_t(r) * 2 * kAtomC;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = oct_col() + 32 * j;
            const float4 y = fma4(x.v[j], ts.v[j], tb.v[j]);
            const float4 hi = make_float4(round_bf(y.x), round_bf(y.y), round_bf(y.z), round_bf(y.w));
            store_bf4(o + c, hi);
            store_bf4(o + kAtomC + c, make_float4(y.x - hi.x, y.y - hi.y, y.z - hi.z, y.w - hi.w));
        }
    }
}
// the encoder's tail: SKIP = qa·QMASK (f32), ABF = bf16(SKIP) (reference: src/diffusion/atom_mlp.cuh:576-591)
__device__ __forceinline__ void atom_tail_skip_rows(const KP& p, int first, int end) {
    for (int i = 0; i < oct_steps(first, end); i++) {
        const int r = min(oct_row(first, i), end - 1);
        const float m = p.geo.qmask[r % p.A];
        const Oct x = oct_load(p.buf.qa + size_t(r) * kAtomC);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = oct_col() + 32 * j;
            const float4 y = make_float4(x.v[j].x * m, x.v[j].y * m, x.v[j].z * m, x.v[j].w * m);
            *reinterpret_cast<float4*>(p.buf.skip + size_t(r) * kAtomC + c) = y;
            store_bf4(p.buf.abf + size_t(r) * kAtomC + c, y);
        }
    }
}
// the decoder's tail: upd = LN(qa·QMASK) @ WUPDᵀ + UPD_B (reference: src/diffusion/atom_mlp.cuh:592-611)
__device__ __forceinline__ void atom_tail_update_rows(const KP& p, int first, int end) {
    for (int i = 0; i < oct_steps(first, end); i++) {
        const int r = min(oct_row(first, i), end - 1);
        const float m = p.geo.qmask[r % p.A];
        Oct x = oct_load(p.buf.qa + size_t(r) * kAtomC);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            x.v[j] = make_float4(x.v[j].x * m, x.v[j].y * m, x.v[j].z * m, x.v[j].w * m);
        }
        oct_layernorm(x, kLnEps);
#pragma unroll
        for (int k = 0; k < kXyz; k++) {
            float u = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 wv = ld4(p.geo.wupd + k * kAtomC + oct_col() + 32 * j);
                u += x.v[j].x * wv.x + x.v[j].y * wv.y + x.v[j].z * wv.z + x.v[j].w * wv.w;
            }
            u = oct_sum(u);
            if ((lane_id() & 7) == 0) {
                p.buf.upd[size_t(r) * kXyz + k] = u + p.geo.upd_b[k];
            }
        }
    }
}
// QKNORM on the atom side: LayerNorm of q (first half of AQG's row) and of k (first half of AKV's)
// over the 128 channels with the block's scale and offset rows. The reference normalises the f32
// accumulators inside its fused projection (src/diffusion/atom_mlp.cuh:306-313, :366-392); here the
// projections are GEMMs with a bf16 epilogue, so this pass reads the rounded q and k.
__device__ __forceinline__ void atom_qknorm_rows(const KP& p, const AtomW& w, int b, int first, int end) {
    const float* qkn = w.qkn + size_t(b) * kQkNormRows * kAtomC;
    for (int i = 0; i < oct_steps(first, end); i++) {
        const int r = min(oct_row(first, i), end - 1);
#pragma unroll
        for (int k = 0; k < 2; k++) {
            bf16* row = (k ? p.buf.akv : p.buf.aqg) + size_t(r) * 2 * kAtomC;
            Oct x;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                x.v[j] = bf4(row + oct_col() + 32 * j);
            }
            oct_layernorm(x, kLnEps);
            const Oct s = oct_load(qkn + (k ? QKN_K_SCALE : QKN_Q_SCALE) * kAtomC), o = oct_load(qkn + (k ? QKN_K_OFFSET : QKN_Q_OFFSET) * kAtomC);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                store_bf4(row + oct_col() + 32 * j, fma4(x.v[j], s.v[j], o.v[j]));
            }
        }
    }
}
// the same passes over all atom rows of the launch, 32 rows (four per warp) to a CTA item
#define CCK_ATOM_ROWS_PHASE(name, call)                                        \
    do {                                                                       \
        const int rows_ = p.S * p.A, items_ = cdiv(rows_, 4 * kWarps);         \
        for (int it_ = d.first(); it_ < items_; it_ += gridDim.x) {            \
            const int f_ = it_ * 4 * kWarps, e_ = min(rows_, f_ + 4 * kWarps); \
            call;                                                              \
        }                                                                      \
        d.advance(items_);                                                     \
    } while (0)
__device__ CCK_PHASE_FN void atom_ln_qk(const KP& p, Deal& d, const AtomW& w, int b) {
    CCK_ATOM_ROWS_PHASE(atom_ln_qk, atom_ln_qk_rows(p, w, b, f_, e_));
}
__device__ CCK_PHASE_FN void atom_ln_t(const KP& p, Deal& d, const AtomW& w, int b) {
    CCK_ATOM_ROWS_PHASE(atom_ln_t, atom_ln_t_rows(p, w, b, f_, e_));
}
__device__ CCK_PHASE_FN void atom_qknorm(const KP& p, Deal& d, const AtomW& w, int b) {
    CCK_ATOM_ROWS_PHASE(atom_qknorm, atom_qknorm_rows(p, w, b, f_, e_));
}
__device__ CCK_PHASE_FN void atom_tail_skip(const KP& p, Deal& d) {
    CCK_ATOM_ROWS_PHASE(atom_tail_skip, atom_tail_skip_rows(p, f_, e_));
}
__device__ CCK_PHASE_FN void atom_tail_update(const KP& p, Deal& d) {
    CCK_ATOM_ROWS_PHASE(atom_tail_update, atom_tail_update_rows(p, f_, e_));
}

// qa = (skip + tb[token of a])·QMASK (reference: src/diffusion/rows.cuh:246-261)
__device__ CCK_PHASE_FN void decoder_init(const KP& p, Deal& d) {
    const int rows = p.S * p.A;
    const int c = 4 * lane_id();
    for (int r = row_first(d); r < rows; r += row_step()) {
        const int s = r / p.A, a = r % p.A;
        const int slot = p.geo.tok2q[a];
        const float m = p.geo.qmask[a];
        float4 x = ld4(p.buf.skip + size_t(r) * kAtomC + c);
        if (slot >= 0) {
            const float4 t = ld4(p.buf.tb + (size_t(s) * p.N + slot / kSlots) * kAtomC + c);
            x.x += t.x, x.y += t.y, x.z += t.z, x.w += t.w;
        }
        *reinterpret_cast<float4*>(p.buf.qa + size_t(r) * kAtomC + c) = make_float4(x.x * m, x.y * m, x.z * m, x.w * m);
    }
    rows_done(d, rows);
}

} // namespace cck

// The sampler's own state: the EDM/Karras level of a step, Philox-keyed noise, centring, random
// rigid augmentation, the Euler update, the atom input features and the final output.
// Cross-CTA sums go through fixed chunks of kChunk slots added in a fixed order, so a fold is
// bit-reproducible run to run.
// Reference for the math: src/diffusion/rng.cuh:8-80, src/diffusion/positions.cuh:42-221, :393-465.
#pragma once

#include "rows.cuh"

namespace cck {

// ---- counter-based RNG: Philox4x32-10, counter (idx, step, sample, stream), key = seed
enum Stream : uint32_t { STREAM_CHURN = 0, STREAM_AUGMENT = 1, STREAM_INIT = 2 };

__host__ __device__ inline void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint64_t m0 = uint64_t(0xD2511F53u) * c[0], m1 = uint64_t(0xCD9E8D57u) * c[2];
        const uint32_t n0 = uint32_t(m1 >> 32) ^ c[1] ^ k0, n2 = uint32_t(m0 >> 32) ^ c[3] ^ k1;
        c[1] = uint32_t(m1), c[3] = uint32_t(m0), c[0] = n0, c[2] = n2;
        k0 += 0x9E3779B9u, k1 += 0xBB67AE85u;
    }
}
// four standard normals by Box-Muller on the 24 high bits of each word
__device__ inline void normals4(uint32_t idx, uint32_t step, uint32_t sample, uint32_t stream, uint32_t k0,
                                uint32_t k1, float (&z)[4]) {
    uint32_t c[4] = {idx, step, sample, stream};
    philox4x32_10(c, k0, k1);
    constexpr float kU = 1.0f / (1 << 24), kTwoPi = 6.2831853071795864f;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const float u1 = float((c[2 * j] >> 8) + 1) * kU, u2 = float(c[2 * j + 1] >> 8) * kU;
        const float r = sqrtf(-2.f * logf(u1)), th = kTwoPi * u2;
        z[2 * j] = r * cosf(th);
        z[2 * j + 1] = r * sinf(th);
    }
}
struct Rigid {
    float r[3][3]; // rows e0, e1, e2: out_j = Σ_i d_i r[i][j]
    float t[3];
};
__device__ __forceinline__ float norm3f(const float* v) {
    return fmaxf(sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]), 1e-10f);
}
// a rotation by Gram-Schmidt on two normal vectors plus a normal translation, from 12 normals
__device__ inline Rigid random_rigid(uint32_t step, uint32_t sample, uint32_t k0, uint32_t k1) {
    float z[12];
    for (int i = 0; i < 3; i++) {
        float n[4];
        normals4(i, step, sample, STREAM_AUGMENT, k0, k1, n);
        for (int j = 0; j < 4; j++) {
            z[4 * i + j] = n[j];
        }
    }
    Rigid g;
    const float n0 = norm3f(z);
    for (int i = 0; i < 3; i++) {
        g.r[0][i] = z[i] / n0;
    }
    const float dd = z[3] * g.r[0][0] + z[4] * g.r[0][1] + z[5] * g.r[0][2];
    float v1[3];
    for (int i = 0; i < 3; i++) {
        v1[i] = z[3 + i] - dd * g.r[0][i];
    }
    const float n1 = norm3f(v1);
    for (int i = 0; i < 3; i++) {
        g.r[1][i] = v1[i] / n1;
    }
    g.r[2][0] = g.r[0][1] * g.r[1][2] - g.r[0][2] * g.r[1][1];
    g.r[2][1] = g.r[0][2] * g.r[1][0] - g.r[0][0] * g.r[1][2];
    g.r[2][2] = g.r[0][0] * g.r[1][1] - g.r[0][1] * g.r[1][0];
    for (int i = 0; i < 3; i++) {
        g.t[i] = z[6 + i];
    }
    return g;
}

// the seed: from the device-side ext block when the caller passes one (the operator path), else
// from the parameter block
__device__ __forceinline__ uint32_t seed_lo(const KP& p) {
    return p.ext ? uint32_t(p.ext[3]) : p.seed_lo;
}
__device__ __forceinline__ uint32_t seed_hi(const KP& p) {
    return p.ext ? uint32_t(p.ext[4]) : p.seed_hi;
}

// ---- the noise levels of one step
struct StepNoise {
    float sigma, t_hat, noise;
};
__device__ inline StepNoise step_noise(const KP& p, int step) {
    const float* misc = p.geo.misc;
    const float sigma = p.tw.sigma[step], prev = p.tw.sigma[step - 1];
    const bool heun = p.flags & F_HEUN;
    float gamma;
    if (heun) {
        gamma = prev >= kChurnMin && prev <= kChurnMax ? misc[M_CHURN] : 0.f;
    } else {
        gamma = sigma > misc[M_GAMMA_MIN] ? misc[M_GAMMA0] : 0.f;
    }
    const float t_hat = prev * (1.f + gamma);
    return {sigma, t_hat, misc[M_NOISE_SCALE] * sqrtf(fmaxf(heun ? kHeunFloor : 0.f, t_hat * t_hat - prev * prev))};
}

constexpr int kSlotsPerThread = (kChunk + kThreads - 1) / kThreads;

__device__ __forceinline__ int nslots(const KP& p) {
    return p.N * kSlots;
}
__device__ __forceinline__ size_t pos_index(const KP& p, int s, int slot) {
    return (size_t(s) * nslots(p) + slot) * kXyz;
}

// pos = σ_0 · z
__device__ CCK_PHASE_FN void positions_init(const KP& p, Deal& d) {
    const int n = p.S * nslots(p), items = cdiv(n, kThreads);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int i = it * kThreads + threadIdx.x;
        if (i < n) {
            const int s = i / nslots(p), slot = i % nslots(p);
            float z[4];
            normals4(slot, 0, s, STREAM_INIT, seed_lo(p), seed_hi(p), z);
            for (int j = 0; j < kXyz; j++) {
                p.buf.pos[pos_index(p, s, slot) + j] = p.tw.sigma[0] * z[j];
            }
        }
    }
    d.advance(items);
}

// K sums over the CTA in a fixed order
template <int K> __device__ void block_reduce(float (&v)[K], float* red) {
#pragma unroll
    for (int k = 0; k < K; k++) {
        v[k] = warp_sum(v[k]);
    }
    __syncthreads();
    if (lane_id() == 0) {
        for (int k = 0; k < K; k++) {
            red[warp_id() * K + k] = v[k];
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < K; k++) {
        v[k] = 0.f;
        for (int w = 0; w < kWarps; w++) {
            v[k] += red[w * K + k];
        }
    }
}

// per (sample, chunk): Σ w·pos and Σ w into CEN
__device__ CCK_PHASE_FN void positions_centre(const KP& p, Deal& d) {
    const int items = p.S * p.chunks;
    float* red = reinterpret_cast<float*>(smem_base());
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int s = it / p.chunks, c = it % p.chunks;
        float v[kCenSums] = {};
        for (int i = 0; i < kSlotsPerThread; i++) {
            const int in_chunk = i * kThreads + threadIdx.x, slot = c * kChunk + in_chunk;
            if (in_chunk < kChunk && slot < nslots(p)) {
                const float w = p.geo.atom_mask[slot];
                const float* q = p.buf.pos + pos_index(p, s, slot);
                v[0] += w * q[0], v[1] += w * q[1], v[2] += w * q[2], v[3] += w;
            }
        }
        block_reduce(v, red);
        if (threadIdx.x < kCenSums) {
            p.buf.cen[size_t(it) * kCenSums + threadIdx.x] = v[threadIdx.x];
        }
    }
    d.advance(items);
}

// xn = ((pos - centre)·R + τ)·mask + noise·z
__device__ CCK_PHASE_FN void positions_augment(const KP& p, Deal& d, int step) {
    const int items = p.S * p.chunks;
    const StepNoise sn = step_noise(p, step);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int s = it / p.chunks, c = it % p.chunks;
        float sum[kCenSums] = {};
        for (int k = 0; k < p.chunks; k++) {
            for (int j = 0; j < kCenSums; j++) {
                sum[j] += p.buf.cen[(size_t(s) * p.chunks + k) * kCenSums + j];
            }
        }
        const float wsum = fmaxf(sum[3], 1e-6f);
        const float centre[kXyz] = {sum[0] / wsum, sum[1] / wsum, sum[2] / wsum};
        const Rigid g = random_rigid(step, s, seed_lo(p), seed_hi(p));
        for (int i = 0; i < kSlotsPerThread; i++) {
            const int in_chunk = i * kThreads + threadIdx.x, slot = c * kChunk + in_chunk;
            if (in_chunk >= kChunk || slot >= nslots(p)) {
                continue;
            }
            const float w = p.geo.atom_mask[slot];
            const float* q = p.buf.pos + pos_index(p, s, slot);
            const float dp[kXyz] = {q[0] - centre[0], q[1] - centre[1], q[2] - centre[2]};
            float z[4];
            normals4(slot, step, s, STREAM_CHURN, seed_lo(p), seed_hi(p), z);
            float* x = p.buf.xn + pos_index(p, s, slot);
            for (int j = 0; j < kXyz; j++) {
                const float rot = dp[0] * g.r[0][j] + dp[1] * g.r[1][j] + dp[2] * g.r[2][j];
                x[j] = (rot + g.t[j]) * w + sn.noise * z[j];
            }
        }
    }
    d.advance(items);
}

// What follows a denoiser call (reference: src/diffusion/positions.cuh:145-221), with
// den = (c_skip·xn + c_out·upd[Q2TA])·mask at the call's noise level:
//   EULER  pos = xn + step_scale·(σ - t̂)·(xn - den)/t̂
//   OUT    mode 1: den into OUT
//   HEUN1  d1 = (xn - den)/t̂ into GRAD, x1 = xn + (σ - t̂)·d1 into XN
//   HEUN2  pos = x1 + (σ - t̂)·((x1 - den2)/σ + d1)/2, den2 taken at σ
enum Update { UPDATE_EULER, UPDATE_OUT, UPDATE_HEUN1, UPDATE_HEUN2 };
__device__ CCK_PHASE_FN void positions_update(const KP& p, Deal& d, int step, int kind) {
    const int n = p.S * nslots(p), items = cdiv(n, kThreads);
    const StepNoise sn = kind == UPDATE_OUT ? StepNoise{0.f, p.t, 0.f} : step_noise(p, step);
    const float dt = sn.sigma - sn.t_hat, t = kind == UPDATE_HEUN2 ? sn.sigma : sn.t_hat;
    const float sd2 = kSigmaData * kSigmaData;
    const float c_skip = sd2 / (t * t + sd2), c_out = t * kSigmaData / sqrtf(t * t + sd2);
    const float step_scale = p.geo.misc[M_STEP_SCALE];
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int i = it * kThreads + threadIdx.x;
        if (i >= n) {
            continue;
        }
        const int s = i / nslots(p), slot = i % nslots(p);
        const int a = p.geo.q2ta[slot];
        const float w = p.geo.atom_mask[slot];
        const size_t pi = pos_index(p, s, slot);
        for (int j = 0; j < kXyz; j++) {
            const float x = p.buf.xn[pi + j];
            const float u = a >= 0 ? p.buf.upd[(size_t(s) * p.A + a) * kXyz + j] : 0.f;
            const float den = (c_skip * x + c_out * u) * w;
            if (kind == UPDATE_OUT) {
                p.buf.out[pi + j] = den;
            } else if (kind == UPDATE_EULER) {
                p.buf.pos[pi + j] = x + step_scale * dt * (x - den) / sn.t_hat;
            } else if (kind == UPDATE_HEUN1) {
                const float d1 = (x - den) / sn.t_hat;
                p.buf.grad[pi + j] = d1;
                p.buf.xn[pi + j] = x + dt * d1;
            } else {
                p.buf.pos[pi + j] = x + dt * ((x - den) / sn.sigma + p.buf.grad[pi + j]) / 2.f;
            }
        }
    }
    d.advance(items);
}

// qa = ((xn·mask/√(t² + σd²)) @ WPOS)·QMASK + SCQ
__device__ CCK_PHASE_FN void atom_init(const KP& p, Deal& d, float t) {
    const int rows = p.S * p.A;
    const float scale = 1.f / sqrtf(t * t + kSigmaData * kSigmaData);
    const int c = 4 * lane_id();
    for (int r = row_first(d); r < rows; r += row_step()) {
        const int s = r / p.A, a = r % p.A, slot = p.geo.tok2q[a];
        float x[kXyz] = {};
        if (slot >= 0) {
            const float* q = p.buf.xn + pos_index(p, s, slot);
            const float w = p.geo.atom_mask[slot];
            for (int j = 0; j < kXyz; j++) {
                x[j] = q[j] * w * scale;
            }
        }
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < kXyz; j++) {
            const float4 wp = ld4(p.geo.wpos + j * kAtomC + c);
            f = make_float4(f.x + x[j] * wp.x, f.y + x[j] * wp.y, f.z + x[j] * wp.z, f.w + x[j] * wp.w);
        }
        const float m = p.geo.qmask[a];
        const float4 q = ld4(p.geo.scq + size_t(a) * kAtomC + c);
        *reinterpret_cast<float4*>(p.buf.qa + size_t(r) * kAtomC + c) =
            make_float4(f.x * m + q.x, f.y * m + q.y, f.z * m + q.z, f.w * m + q.w);
    }
    rows_done(d, rows);
}

// the operator's result: positions [S][Nb][24][3], zero past the real tokens
__device__ CCK_PHASE_FN void positions_output(const KP& p, Deal& d) {
    if (!p.out) {
        return;
    }
    const int per = p.out_tokens * kSlots * kXyz, n = p.S * per, items = cdiv(n, kThreads);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int i = it * kThreads + threadIdx.x;
        if (i < n) {
            const int s = i / per, j = i % per;
            p.out[i] = j < nslots(p) * kXyz ? p.buf.pos[size_t(s) * nslots(p) * kXyz + j] : 0.f;
        }
    }
    d.advance(items);
}

} // namespace cck

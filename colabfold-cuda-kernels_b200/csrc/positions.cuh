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

// REALIGN, first half: den into GRAD and, per (sample, chunk), the moments of the rigid alignment of
// xn onto den into KAB: Σw, Σw·x, Σw·den, Σw·x·denᵀ (reference: src/diffusion/positions.cuh:166-219)
__device__ CCK_PHASE_FN void positions_moments(const KP& p, Deal& d, int step) {
    const int items = p.S * p.chunks;
    float* red = reinterpret_cast<float*>(smem_base());
    const float t = step_noise(p, step).t_hat, sd2 = kSigmaData * kSigmaData;
    const float c_skip = sd2 / (t * t + sd2), c_out = t * kSigmaData / sqrtf(t * t + sd2);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int s = it / p.chunks, c = it % p.chunks;
        float m[kMoments] = {};
        for (int i = 0; i < kSlotsPerThread; i++) {
            const int in_chunk = i * kThreads + threadIdx.x, slot = c * kChunk + in_chunk;
            if (in_chunk >= kChunk || slot >= nslots(p)) {
                continue;
            }
            const int a = p.geo.q2ta[slot];
            const float w = p.geo.atom_mask[slot];
            const size_t pi = pos_index(p, s, slot);
            float x[kXyz], den[kXyz];
            for (int j = 0; j < kXyz; j++) {
                x[j] = p.buf.xn[pi + j];
                const float u = a >= 0 ? p.buf.upd[(size_t(s) * p.A + a) * kXyz + j] : 0.f;
                den[j] = (c_skip * x[j] + c_out * u) * w;
                p.buf.grad[pi + j] = den[j];
            }
            m[0] += w;
            for (int j = 0; j < kXyz; j++) {
                m[1 + j] += w * x[j];
                m[4 + j] += w * den[j];
                for (int k = 0; k < kXyz; k++) {
                    m[7 + 3 * j + k] += w * x[j] * den[k];
                }
            }
        }
        block_reduce(m, red);
        if (threadIdx.x < kMoments) {
            p.buf.kab[size_t(it) * kMoments + threadIdx.x] = m[threadIdx.x];
        }
    }
    d.advance(items);
}
// The eigenvector of the largest eigenvalue of a symmetric 4x4 matrix by cyclic Jacobi sweeps
// (reference: src/diffusion/positions.cuh:223-263)
__device__ inline void top_eigenvector(float (&a)[4][4], float (&q)[4]) {
    float v[4][4] = {{1, 0, 0, 0}, {0, 1, 0, 0}, {0, 0, 1, 0}, {0, 0, 0, 1}};
    for (int sweep = 0; sweep < kJacobiSweeps; sweep++) {
        float off = 0.f;
        for (int i = 0; i < 4; i++) {
            for (int j = i + 1; j < 4; j++) {
                off += a[i][j] * a[i][j];
            }
        }
        if (off < kTiny) {
            break;
        }
        for (int i = 0; i < 4; i++) {
            for (int j = i + 1; j < 4; j++) {
                if (fabsf(a[i][j]) < kTiny) {
                    continue;
                }
                const float theta = (a[j][j] - a[i][i]) / (2.f * a[i][j]);
                const float tn = copysignf(1.f, theta) / (fabsf(theta) + sqrtf(theta * theta + 1.f));
                const float cs = 1.f / sqrtf(tn * tn + 1.f), sn = tn * cs;
                for (int k = 0; k < 4; k++) { // columns i, j
                    const float x = a[k][i], y = a[k][j];
                    a[k][i] = cs * x - sn * y, a[k][j] = sn * x + cs * y;
                }
                for (int k = 0; k < 4; k++) { // rows i, j
                    const float x = a[i][k], y = a[j][k];
                    a[i][k] = cs * x - sn * y, a[j][k] = sn * x + cs * y;
                }
                for (int k = 0; k < 4; k++) { // the accumulated rotation
                    const float x = v[k][i], y = v[k][j];
                    v[k][i] = cs * x - sn * y, v[k][j] = sn * x + cs * y;
                }
            }
        }
    }
    int best = 0;
    for (int i = 1; i < 4; i++) {
        best = a[i][i] > a[best][best] ? i : best;
    }
    for (int k = 0; k < 4; k++) {
        q[k] = v[k][best];
    }
}
// REALIGN, second half: xn aligned rigidly onto den (Horn's quaternion method on the weighted
// cross-covariance), then the Euler step from the aligned xn (reference: src/diffusion/positions.cuh:265-336)
__device__ CCK_PHASE_FN void positions_realign(const KP& p, Deal& d, int step) {
    const int items = p.S * p.chunks;
    float* rt = reinterpret_cast<float*>(smem_base()); // R as used on row vectors [3][3], then x̄ and d̄
    const StepNoise sn = step_noise(p, step);
    const float dt = sn.sigma - sn.t_hat, step_scale = p.geo.misc[M_STEP_SCALE];
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int s = it / p.chunks, c = it % p.chunks;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m[kMoments] = {};
            for (int k = 0; k < p.chunks; k++) {
                for (int j = 0; j < kMoments; j++) {
                    m[j] += p.buf.kab[(size_t(s) * p.chunks + k) * kMoments + j];
                }
            }
            const float w = m[0];
            float h[kXyz][kXyz]; // Σ w (x - x̄)(d - d̄)ᵀ
            for (int i = 0; i < kXyz; i++) {
                for (int j = 0; j < kXyz; j++) {
                    h[i][j] = m[7 + 3 * i + j] - m[1 + i] * m[4 + j] / w;
                }
            }
            float n[4][4] = {{h[0][0] + h[1][1] + h[2][2], h[1][2] - h[2][1], h[2][0] - h[0][2], h[0][1] - h[1][0]},
                             {h[1][2] - h[2][1], h[0][0] - h[1][1] - h[2][2], h[0][1] + h[1][0], h[2][0] + h[0][2]},
                             {h[2][0] - h[0][2], h[0][1] + h[1][0], -h[0][0] + h[1][1] - h[2][2], h[1][2] + h[2][1]},
                             {h[0][1] - h[1][0], h[2][0] + h[0][2], h[1][2] + h[2][1], -h[0][0] - h[1][1] + h[2][2]}};
            float q[4];
            top_eigenvector(n, q);
            const float q0 = q[0], q1 = q[1], q2 = q[2], q3 = q[3];
            // r maps x - x̄ onto d - d̄ as column vectors; stored transposed for row vectors
            const float r[kXyz][kXyz] = {{q0 * q0 + q1 * q1 - q2 * q2 - q3 * q3, 2 * (q1 * q2 - q0 * q3), 2 * (q1 * q3 + q0 * q2)},
                                         {2 * (q1 * q2 + q0 * q3), q0 * q0 - q1 * q1 + q2 * q2 - q3 * q3, 2 * (q2 * q3 - q0 * q1)},
                                         {2 * (q1 * q3 - q0 * q2), 2 * (q2 * q3 + q0 * q1), q0 * q0 - q1 * q1 - q2 * q2 + q3 * q3}};
            for (int i = 0; i < kXyz; i++) {
                for (int j = 0; j < kXyz; j++) {
                    rt[i * kXyz + j] = r[j][i];
                }
                rt[9 + i] = m[1 + i] / w;
                rt[12 + i] = m[4 + i] / w;
            }
        }
        __syncthreads();
        for (int i = 0; i < kSlotsPerThread; i++) {
            const int in_chunk = i * kThreads + threadIdx.x, slot = c * kChunk + in_chunk;
            if (in_chunk >= kChunk || slot >= nslots(p)) {
                continue;
            }
            const size_t pi = pos_index(p, s, slot);
            const float* x = p.buf.xn + pi;
            const float dx[kXyz] = {x[0] - rt[9], x[1] - rt[10], x[2] - rt[11]};
            for (int j = 0; j < kXyz; j++) {
                const float al = dx[0] * rt[j] + dx[1] * rt[kXyz + j] + dx[2] * rt[2 * kXyz + j] + rt[12 + j];
                p.buf.pos[pi + j] = al + step_scale * dt * (al - p.buf.grad[pi + j]) / sn.t_hat;
            }
        }
    }
    __syncthreads();
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
__device__ __forceinline__ float dot3(const float* a, const float* b) {
    return a[0] * b[0] + a[1] * b[1] + a[2] * b[2];
}
__device__ __forceinline__ void cross3(const float* a, const float* b, float* o) {
    o[0] = a[1] * b[2] - a[2] * b[1], o[1] = a[2] * b[0] - a[0] * b[2], o[2] = a[0] * b[1] - a[1] * b[0];
}
// CHIRAL: the gradient of (improper dihedral of p0..p3 - ideal)² with respect to the atom playing
// `role`, by reverse differentiation of the dihedral's construction (reference:
// src/diffusion/positions.cuh:351-390)
__device__ __noinline__ void chiral_grad(const float (&p)[4][kXyz], float ideal, int role, float* out) {
    float b0[3], b1[3], b2[3], u[3], v[3], w[3];
    for (int i = 0; i < 3; i++) {
        b0[i] = p[0][i] - p[1][i], b1[i] = p[2][i] - p[1][i], b2[i] = p[3][i] - p[2][i];
    }
    const float n1 = sqrtf(dot3(b1, b1)), nb = n1 + kChiralEps;
    for (int i = 0; i < 3; i++) {
        u[i] = b1[i] / nb;
    }
    const float b0u = dot3(b0, u), b2u = dot3(b2, u);
    for (int i = 0; i < 3; i++) {
        v[i] = b0[i] - b0u * u[i], w[i] = b2[i] - b2u * u[i];
    }
    float uv[3], wu[3], vw[3];
    cross3(u, v, uv), cross3(w, u, wu), cross3(v, w, vw);
    const float y = dot3(uv, w) + kChiralEps, x = dot3(v, w) + kChiralEps;
    // back through phi = atan2(y, x)
    const float g = 2.f * (atan2f(y, x) - ideal), r2 = x * x + y * y;
    const float gy = g * x / r2, gx = -g * y / r2;
    // through y = (u x v)·w and x = v·w
    float gv[3], gw[3], gu[3];
    for (int i = 0; i < 3; i++) {
        gv[i] = gy * wu[i] + gx * w[i];
        gw[i] = gy * uv[i] + gx * v[i];
        gu[i] = gy * vw[i];
    }
    // through the projections v = b0 - (b0·u)u, w = b2 - (b2·u)u
    const float gvu = dot3(gv, u), gwu = dot3(gw, u);
    float gb0[3], gb1[3], gb2[3];
    for (int i = 0; i < 3; i++) {
        gb0[i] = gv[i] - gvu * u[i];
        gb2[i] = gw[i] - gwu * u[i];
        gu[i] -= gvu * b0[i] + b0u * gv[i] + gwu * b2[i] + b2u * gw[i];
    }
    // through u = b1 / (|b1| + eps)
    const float gub1 = dot3(gu, b1);
    for (int i = 0; i < 3; i++) {
        gb1[i] = gu[i] / nb - b1[i] * gub1 / (nb * nb * fmaxf(n1, 1e-30f));
    }
    // b0 = p0 - p1, b1 = p2 - p1, b2 = p3 - p2
    for (int i = 0; i < 3; i++) {
        const float r[4] = {gb0[i], -gb0[i] - gb1[i], gb1[i] - gb2[i], gb2[i]};
        out[i] = r[role];
    }
}
__device__ CCK_PHASE_FN void atom_init(const KP& p, Deal& d, float t) {
    const int rows = p.S * p.A;
    const float scale = 1.f / sqrtf(t * t + kSigmaData * kSigmaData);
    const int c = 4 * lane_id();
    for (int r = row_first(d); r < rows; r += row_step()) {
        const int s = r / p.A, a = r % p.A, slot = p.geo.tok2q[a];
        float x[kXyz] = {}, gr[kXyz] = {};
        if (slot >= 0) {
            const float* q = p.buf.xn + pos_index(p, s, slot);
            const float w = p.geo.atom_mask[slot];
            for (int j = 0; j < kXyz; j++) {
                x[j] = q[j] * w * scale;
            }
            if (p.flags & F_CHIRAL) { // the chirality restraints this atom takes part in (reference: src/diffusion/positions.cuh:406-430)
                for (int e = p.geo.chir_ptr[slot]; e < p.geo.chir_ptr[slot + 1]; e++) {
                    const int centre = p.geo.chir_idx[e] / 4, role = p.geo.chir_idx[e] % 4;
                    const float ideal = p.geo.chir_a[centre];
                    if (ideal == 0.f) {
                        continue;
                    }
                    float p4[4][kXyz], gi[kXyz];
                    for (int k = 0; k < 4; k++) {
                        const int sk = p.geo.chir_c[centre * 4 + k];
                        const float* pk = p.buf.xn + pos_index(p, s, sk);
                        for (int j = 0; j < kXyz; j++) {
                            p4[k][j] = pk[j] * p.geo.atom_mask[sk] * scale;
                        }
                    }
                    chiral_grad(p4, ideal, role, gi);
                    for (int j = 0; j < kXyz; j++) {
                        gr[j] += gi[j];
                    }
                }
                for (int j = 0; j < kXyz; j++) {
                    gr[j] = isfinite(gr[j]) ? gr[j] : 0.f;
                }
            }
        }
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < kXyz; j++) {
            const float4 wp = ld4(p.geo.wpos + j * kAtomC + c);
            f = make_float4(f.x + x[j] * wp.x, f.y + x[j] * wp.y, f.z + x[j] * wp.z, f.w + x[j] * wp.w);
            if (p.flags & F_CHIRAL) {
                const float4 wc = ld4(p.geo.chir_w + j * kAtomC + c);
                f = make_float4(f.x + gr[j] * wc.x, f.y + gr[j] * wc.y, f.z + gr[j] * wc.z, f.w + gr[j] * wc.w);
            }
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

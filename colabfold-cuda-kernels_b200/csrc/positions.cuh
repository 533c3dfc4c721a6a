// The sampler's own state between denoiser calls: the noise level of a step, Philox-keyed normals,
// centring, the random rigid motion, the Euler / Heun / aligned updates, the atom input features and
// the operator's result.
//
// Layout: positions live per slot (24 slots per token), [sample][slot][xyz] f32. A warp works on a
// tile of 32 consecutive slots, one per lane: 384 contiguous bytes that 24 lanes move with one 128-bit
// access each and a shared-memory stage turns into three floats per lane. Sums over a sample go
// through per-chunk partial sums (CEN, KAB; a chunk is kChunk slots = 32 tiles) that are added in chunk
// order, and inside a chunk in a fixed lane / warp order, so a fold is bit-reproducible.
// What is fixed by the operator's contract and restated here: the Philox counter (slot, step, sample,
// stream) with the seed as key, the Box-Muller form on the 24 high bits, the chunk size, and the
// formulas (reference: src/diffusion/rng.cuh:8-80, src/diffusion/positions.cuh:42-221, :223-336, :351-465).
#pragma once

#include "rows.cuh"

namespace cck {

// ---- Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): ten rounds of two
// 32 x 32 -> 64 bit multiplications with the key bumped by the Weyl constants after each round
enum Stream : uint32_t { STREAM_CHURN = 0, STREAM_AUGMENT = 1, STREAM_INIT = 2 };

struct PhiloxWords {
    uint32_t w[4];
};
__host__ __device__ inline PhiloxWords philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    constexpr uint32_t kMulA = 0xD2511F53u, kMulB = 0xCD9E8D57u, kWeylA = 0x9E3779B9u, kWeylB = 0xBB67AE85u;
    PhiloxWords s{{c0, c1, c2, c3}};
#pragma unroll
    for (int round = 0; round < 10; round++, k0 += kWeylA, k1 += kWeylB) {
        const uint64_t pa = uint64_t(kMulA) * s.w[0], pb = uint64_t(kMulB) * s.w[2];
        s = PhiloxWords{{uint32_t(pb >> 32) ^ s.w[1] ^ k0, uint32_t(pb), uint32_t(pa >> 32) ^ s.w[3] ^ k1, uint32_t(pa)}};
    }
    return s;
}
// Four standard normals of one counter: Box-Muller on word pairs (0, 1) and (2, 3), uniforms from the
// 24 high bits, the first of a pair kept away from zero
struct Normals4 {
    float z[4];
};
__device__ inline Normals4 philox_normals(uint32_t idx, uint32_t step, uint32_t sample, uint32_t stream, uint32_t k0, uint32_t k1) {
    const PhiloxWords s = philox(idx, step, sample, stream, k0, k1);
    constexpr float kInv24 = 1.0f / 16777216.f, kTwoPi = 6.2831853071795864f;
    Normals4 n;
#pragma unroll
    for (int pair = 0; pair < 2; pair++) {
        const float u = float((s.w[2 * pair] >> 8) + 1) * kInv24, v = float(s.w[2 * pair + 1] >> 8) * kInv24;
        const float radius = sqrtf(-2.f * logf(u)), angle = kTwoPi * v;
        n.z[2 * pair] = radius * cosf(angle), n.z[2 * pair + 1] = radius * sinf(angle);
    }
    return n;
}

// ---- small vectors
struct V3 {
    float x, y, z;
};
__device__ __forceinline__ V3 operator-(V3 a, V3 b) {
    return {a.x - b.x, a.y - b.y, a.z - b.z};
}
__device__ __forceinline__ V3 operator+(V3 a, V3 b) {
    return {a.x + b.x, a.y + b.y, a.z + b.z};
}
__device__ __forceinline__ V3 operator/(V3 a, float s) {
    return {a.x / s, a.y / s, a.z / s};
}
__device__ __forceinline__ V3 operator*(float s, V3 a) {
    return {s * a.x, s * a.y, s * a.z};
}
__device__ __forceinline__ float dot(V3 a, V3 b) {
    return a.x * b.x + a.y * b.y + a.z * b.z;
}
__device__ __forceinline__ V3 cross(V3 a, V3 b) {
    return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x};
}
__device__ __forceinline__ float length_floored(V3 a) {
    return fmaxf(sqrtf(dot(a, a)), 1e-10f);
}

// The random rigid motion of (step, sample): counters 0..2 of the AUGMENT stream give twelve normals;
// the first two triples become an orthonormal frame by Gram-Schmidt, its third axis their cross
// product, the third triple the translation. A row vector d moves to d·R + t with R's rows e0, e1, e2.
struct RigidMotion {
    V3 e0, e1, e2, t;
    __device__ __forceinline__ float apply(V3 d, int axis) const {
        const float a0 = axis == 0 ? e0.x : axis == 1 ? e0.y : e0.z, a1 = axis == 0 ? e1.x : axis == 1 ? e1.y : e1.z;
        const float a2 = axis == 0 ? e2.x : axis == 1 ? e2.y : e2.z, tt = axis == 0 ? t.x : axis == 1 ? t.y : t.z;
        return d.x * a0 + d.y * a1 + d.z * a2 + tt;
    }
};
__device__ inline RigidMotion random_rigid(uint32_t step, uint32_t sample, uint32_t k0, uint32_t k1) {
    const Normals4 a = philox_normals(0, step, sample, STREAM_AUGMENT, k0, k1);
    const Normals4 b = philox_normals(1, step, sample, STREAM_AUGMENT, k0, k1);
    const Normals4 c = philox_normals(2, step, sample, STREAM_AUGMENT, k0, k1);
    const V3 first{a.z[0], a.z[1], a.z[2]}, second{a.z[3], b.z[0], b.z[1]};
    RigidMotion m;
    m.e0 = first / length_floored(first);
    const V3 rest = second - dot(second, m.e0) * m.e0;
    m.e1 = rest / length_floored(rest);
    m.e2 = cross(m.e0, m.e1);
    m.t = V3{b.z[2], b.z[3], c.z[0]};
    return m;
}

// the seed: from the device-side ext block when the caller passes one (the operator path), else
// from the parameter block
__device__ __forceinline__ uint32_t seed_lo(const KP& p) {
    return p.ext ? uint32_t(p.ext[3]) : p.seed_lo;
}
__device__ __forceinline__ uint32_t seed_hi(const KP& p) {
    return p.ext ? uint32_t(p.ext[4]) : p.seed_hi;
}

// ---- the noise levels of one step: σ of the step, the raised level t̂ = σ_prev·(1 + γ) that the
// denoiser sees, and the standard deviation of the noise that lifts σ_prev to t̂. γ is γ0 above the
// γ_min level (Euler), or the churn inside the window [kChurnMin, kChurnMax] of σ_prev (Heun, which
// also keeps the variance off zero).
struct StepNoise {
    float sigma, t_hat, noise;
};
__device__ inline StepNoise step_noise(const KP& p, int step) {
    const float* misc = p.geo.misc;
    const float now = p.tw.sigma[step], before = p.tw.sigma[step - 1];
    const bool heun = (p.flags & F_HEUN) != 0;
    const bool churned = heun ? (before >= kChurnMin && before <= kChurnMax) : (now > misc[M_GAMMA_MIN]);
    const float gamma = churned ? misc[heun ? M_CHURN : M_GAMMA0] : 0.f;
    StepNoise n;
    n.sigma = now, n.t_hat = before * (1.f + gamma);
    n.noise = misc[M_NOISE_SCALE] * sqrtf(fmaxf(heun ? kHeunFloor : 0.f, n.t_hat * n.t_hat - before * before));
    return n;
}
// the denoiser's output scaling at level t: den = c_skip·x + c_out·update
struct EdmScale {
    float c_skip, c_out;
};
__device__ __forceinline__ EdmScale edm_scale(float t) {
    const float var = kSigmaData * kSigmaData, total = t * t + var;
    return {var / total, t * kSigmaData / sqrtf(total)};
}

// ---- tiles: 32 consecutive slots of one sample, one per lane of a warp. In memory a tile is 384
// contiguous bytes: 24 lanes move it with one 128-bit access each, and the warp's staging area in
// shared memory turns that into one slot (three floats) per lane and back. Position buffers are
// [sample][slot][xyz] with 24 slots per token, so a sample starts on a 128-bit boundary and so does
// every tile; the last tile of a sample may be short by a multiple of four slots.
constexpr int kTile = 32, kTileFloats = kTile * kXyz, kTilesPerChunk = kChunk / kTile;
constexpr int kSumScratch = 1024; // bytes at the head of the scratch area for cta_sums; the warps' tile stages follow
static_assert(kSlots % 4 == 0 && kChunk % kTile == 0, "tiles are whole 128-bit accesses and chunks whole tiles");

__device__ __forceinline__ int nslots(const KP& p) {
    return p.N * kSlots;
}
__device__ __forceinline__ float* tile_stage() {
    return reinterpret_cast<float*>(smem_base() + kSumScratch) + warp_id() * kTileFloats;
}
struct Tile {
    int sample, slot0, count; // count = 0: no such tile
    size_t off;               // of the tile's first float in a [sample][slot][xyz] buffer
    __device__ __forceinline__ int slot() const { // this lane's slot
        return slot0 + lane_id();
    }
    __device__ __forceinline__ bool mine() const { // this lane has one
        return lane_id() < count;
    }
};
__device__ __forceinline__ Tile make_tile(const KP& p, int sample, int t) {
    Tile x;
    x.sample = sample, x.slot0 = t * kTile;
    x.count = max(0, min(kTile, nslots(p) - x.slot0));
    x.off = (size_t(sample) * nslots(p) + x.slot0) * kXyz;
    return x;
}
// this lane's slot of the tile (zeros past the tile's end)
__device__ __forceinline__ V3 tile_load(const float* buf, const Tile& t) {
    float* st = tile_stage();
    const int l = lane_id();
    if (4 * l < t.count * kXyz) {
        reinterpret_cast<float4*>(st)[l] = reinterpret_cast<const float4*>(buf + t.off)[l];
    }
    __syncwarp();
    const V3 v = t.mine() ? V3{st[3 * l], st[3 * l + 1], st[3 * l + 2]} : V3{0.f, 0.f, 0.f};
    __syncwarp();
    return v;
}
__device__ __forceinline__ void tile_store(float* buf, const Tile& t, V3 v) {
    float* st = tile_stage();
    const int l = lane_id();
    st[3 * l] = v.x, st[3 * l + 1] = v.y, st[3 * l + 2] = v.z;
    __syncwarp();
    if (4 * l < t.count * kXyz) {
        reinterpret_cast<float4*>(buf + t.off)[l] = reinterpret_cast<const float4*>(st)[l];
    }
    __syncwarp();
}
// Work items. Phases without a sum deal groups of kWarps tiles of one sample (a warp each) over the
// grid; phases that sum deal (sample, chunk) and a warp walks the chunk's tiles w, w + kWarps, ...
__device__ __forceinline__ int tile_groups(const KP& p) {
    return cdiv(cdiv(nslots(p), kTile), kWarps);
}
__device__ __forceinline__ Tile group_tile(const KP& p, int it) {
    const int groups = tile_groups(p), sample = it / groups;
    return make_tile(p, sample, (it - sample * groups) * kWarps + warp_id());
}

// K sums over the CTA, the same in every thread: lanes by butterfly, then the warps' partial sums in
// warp order. Uses the first kSumScratch bytes of the scratch area.
template <int K> __device__ void cta_sums(float (&v)[K]) {
    static_assert(K * kWarps * 4 <= kSumScratch, "the sums' scratch");
    float* scratch = reinterpret_cast<float*>(smem_base());
    __syncthreads(); // the scratch of an earlier call has been read
#pragma unroll
    for (int k = 0; k < K; k++) {
        const float w = warp_sum(v[k]);
        if (lane_id() == 0) {
            scratch[k * kWarps + warp_id()] = w;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < K; k++) {
        float total = 0.f;
        for (int w = 0; w < kWarps; w++) {
            total += scratch[k * kWarps + w];
        }
        v[k] = total;
    }
}
// the per-chunk partial sums of a sample, added in chunk order
template <int K> __device__ __forceinline__ void sample_sums(const float* partial, int sample, int chunks, float (&total)[K]) {
#pragma unroll
    for (int k = 0; k < K; k++) {
        total[k] = 0.f;
    }
    for (int c = 0; c < chunks; c++) {
#pragma unroll
        for (int k = 0; k < K; k++) {
            total[k] += partial[(size_t(sample) * chunks + c) * K + k];
        }
    }
}
// the denoised position of a slot: (c_skip·x + c_out·update of the slot's atom)·mask
__device__ __forceinline__ V3 denoised(const KP& p, EdmScale e, int sample, int atom, float mask, V3 x) {
    V3 u{0.f, 0.f, 0.f};
    if (atom >= 0) {
        const float* q = p.buf.upd + (size_t(sample) * p.A + atom) * kXyz;
        u = V3{q[0], q[1], q[2]};
    }
    return {(e.c_skip * x.x + e.c_out * u.x) * mask, (e.c_skip * x.y + e.c_out * u.y) * mask, (e.c_skip * x.z + e.c_out * u.z) * mask};
}

// ---- phases

// pos = σ_0 · z, z from the INIT stream at step 0
__device__ CCK_PHASE_FN void positions_init(const KP& p, Deal& d) {
    const int items = p.S * tile_groups(p);
    const float sigma0 = p.tw.sigma[0];
    for (int it = d.first(); it < items; it += gridDim.x) {
        const Tile t = group_tile(p, it);
        if (t.count == 0) {
            continue;
        }
        const Normals4 n = philox_normals(t.slot(), 0, t.sample, STREAM_INIT, seed_lo(p), seed_hi(p));
        tile_store(p.buf.pos, t, V3{sigma0 * n.z[0], sigma0 * n.z[1], sigma0 * n.z[2]});
    }
    d.advance(items);
}

// per (sample, chunk): Σ mask·pos and Σ mask into CEN
__device__ CCK_PHASE_FN void positions_centre(const KP& p, Deal& d) {
    const int items = p.S * p.chunks;
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int sample = it / p.chunks, chunk = it - sample * p.chunks;
        float sums[kCenSums] = {0.f, 0.f, 0.f, 0.f};
        for (int tt = warp_id(); tt < kTilesPerChunk; tt += kWarps) {
            const Tile t = make_tile(p, sample, chunk * kTilesPerChunk + tt);
            if (t.count == 0) {
                break;
            }
            const V3 x = tile_load(p.buf.pos, t);
            const float w = t.mine() ? p.geo.atom_mask[t.slot()] : 0.f;
            sums[0] += w * x.x, sums[1] += w * x.y, sums[2] += w * x.z, sums[3] += w;
        }
        cta_sums(sums);
        if (threadIdx.x < kCenSums) {
            p.buf.cen[size_t(it) * kCenSums + threadIdx.x] = sums[threadIdx.x];
        }
    }
    d.advance(items);
}

// xn = ((pos - centre)·R + τ)·mask + noise·z, z from the CHURN stream
__device__ CCK_PHASE_FN void positions_augment(const KP& p, Deal& d, int step) {
    const int items = p.S * tile_groups(p);
    const StepNoise sn = step_noise(p, step);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const Tile t = group_tile(p, it);
        if (t.count == 0) {
            continue;
        }
        float sums[kCenSums];
        sample_sums(p.buf.cen, t.sample, p.chunks, sums);
        const float weight = fmaxf(sums[3], 1e-6f);
        const V3 centre{sums[0] / weight, sums[1] / weight, sums[2] / weight};
        const RigidMotion g = random_rigid(step, t.sample, seed_lo(p), seed_hi(p));
        const V3 rel = tile_load(p.buf.pos, t) - centre;
        const float m = t.mine() ? p.geo.atom_mask[t.slot()] : 0.f;
        const Normals4 n = philox_normals(t.slot(), step, t.sample, STREAM_CHURN, seed_lo(p), seed_hi(p));
        tile_store(p.buf.xn, t, V3{g.apply(rel, 0) * m + sn.noise * n.z[0], g.apply(rel, 1) * m + sn.noise * n.z[1], g.apply(rel, 2) * m + sn.noise * n.z[2]});
    }
    d.advance(items);
}

// What follows a denoiser call, with den = denoised position at the call's noise level
// (reference: src/diffusion/positions.cuh:145-221):
//   EULER  pos = xn + step_scale·(σ - t̂)·(xn - den)/t̂
//   OUT    mode 1: den into OUT
//   HEUN1  d1 = (xn - den)/t̂ into GRAD, x1 = xn + (σ - t̂)·d1 into XN
//   HEUN2  pos = x1 + (σ - t̂)·((x1 - den2)/σ + d1)/2, den2 taken at σ
enum Update { UPDATE_EULER, UPDATE_OUT, UPDATE_HEUN1, UPDATE_HEUN2 };
__device__ CCK_PHASE_FN void positions_update(const KP& p, Deal& d, int step, int kind) {
    const int items = p.S * tile_groups(p);
    const StepNoise sn = kind == UPDATE_OUT ? StepNoise{0.f, p.t, 0.f} : step_noise(p, step);
    const float dt = sn.sigma - sn.t_hat, scale = p.geo.misc[M_STEP_SCALE];
    const EdmScale e = edm_scale(kind == UPDATE_HEUN2 ? sn.sigma : sn.t_hat);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const Tile t = group_tile(p, it);
        if (t.count == 0) {
            continue;
        }
        const V3 x = tile_load(p.buf.xn, t);
        const bool on = t.mine();
        const V3 den = denoised(p, e, t.sample, on ? p.geo.q2ta[t.slot()] : -1, on ? p.geo.atom_mask[t.slot()] : 0.f, x);
        if (kind == UPDATE_OUT) {
            tile_store(p.buf.out, t, den);
        } else if (kind == UPDATE_EULER) {
            tile_store(p.buf.pos, t, V3{x.x + scale * dt * (x.x - den.x) / sn.t_hat, x.y + scale * dt * (x.y - den.y) / sn.t_hat,
                                        x.z + scale * dt * (x.z - den.z) / sn.t_hat});
        } else if (kind == UPDATE_HEUN1) {
            const V3 slope{(x.x - den.x) / sn.t_hat, (x.y - den.y) / sn.t_hat, (x.z - den.z) / sn.t_hat};
            tile_store(p.buf.grad, t, slope);
            tile_store(p.buf.xn, t, V3{x.x + dt * slope.x, x.y + dt * slope.y, x.z + dt * slope.z});
        } else {
            const V3 slope = tile_load(p.buf.grad, t);
            tile_store(p.buf.pos, t, V3{x.x + dt * ((x.x - den.x) / sn.sigma + slope.x) / 2.f, x.y + dt * ((x.y - den.y) / sn.sigma + slope.y) / 2.f,
                                        x.z + dt * ((x.z - den.z) / sn.sigma + slope.z) / 2.f});
        }
    }
    d.advance(items);
}

// REALIGN, first half: den into GRAD and, per (sample, chunk), the weighted moments of the pair
// (xn, den) that the rigid alignment of xn onto den needs, into KAB:
// [Σw, Σw·x (3), Σw·den (3), Σw·x·denᵀ (9, row-major)] (reference: src/diffusion/positions.cuh:166-219)
__device__ CCK_PHASE_FN void positions_moments(const KP& p, Deal& d, int step) {
    const int items = p.S * p.chunks;
    const EdmScale e = edm_scale(step_noise(p, step).t_hat);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int sample = it / p.chunks, chunk = it - sample * p.chunks;
        float mom[kMoments];
#pragma unroll
        for (int i = 0; i < kMoments; i++) {
            mom[i] = 0.f;
        }
        for (int tt = warp_id(); tt < kTilesPerChunk; tt += kWarps) {
            const Tile t = make_tile(p, sample, chunk * kTilesPerChunk + tt);
            if (t.count == 0) {
                break;
            }
            const V3 x = tile_load(p.buf.xn, t);
            const bool on = t.mine();
            const float w = on ? p.geo.atom_mask[t.slot()] : 0.f;
            const V3 den = denoised(p, e, sample, on ? p.geo.q2ta[t.slot()] : -1, w, x);
            tile_store(p.buf.grad, t, den);
            const float xs[kXyz] = {x.x, x.y, x.z}, ds[kXyz] = {den.x, den.y, den.z};
            mom[0] += w;
#pragma unroll
            for (int a = 0; a < kXyz; a++) {
                mom[1 + a] += w * xs[a], mom[4 + a] += w * ds[a];
#pragma unroll
                for (int b = 0; b < kXyz; b++) {
                    mom[7 + 3 * a + b] += w * xs[a] * ds[b];
                }
            }
        }
        cta_sums(mom);
        if (threadIdx.x < kMoments) {
            p.buf.kab[size_t(it) * kMoments + threadIdx.x] = mom[threadIdx.x];
        }
    }
    d.advance(items);
}

// The unit eigenvector of the largest eigenvalue of a symmetric 4 x 4 matrix by cyclic Jacobi
// rotations (Golub & Van Loan, Matrix Computations, section 8.5): every rotation zeroes one
// off-diagonal pair with the stable tangent t = sgn(θ) / (|θ| + √(θ² + 1)), θ = (a_qq - a_pp) / 2a_pq,
// and is applied as the symmetric update of rows and columns p, q; the rotations' product holds the
// eigenvectors. At most kJacobiSweeps sweeps, ended early when the off-diagonal mass is below kTiny
// (the same bounds as the reference, src/diffusion/positions.cuh:16-17).
struct Sym4 {
    float a[4][4];
};
__device__ inline void top_eigenvector(Sym4 m, float (&vec)[4]) {
    float e[4][4]; // columns: the eigenvector estimates
    for (int i = 0; i < 4; i++) {
        for (int j = 0; j < 4; j++) {
            e[i][j] = i == j ? 1.f : 0.f;
        }
    }
    for (int sweep = 0; sweep < kJacobiSweeps; sweep++) {
        float off = 0.f;
        for (int pp = 0; pp < 4; pp++) {
            for (int qq = pp + 1; qq < 4; qq++) {
                off += m.a[pp][qq] * m.a[pp][qq];
            }
        }
        if (off < kTiny) {
            break;
        }
        for (int pp = 0; pp < 3; pp++) {
            for (int qq = pp + 1; qq < 4; qq++) {
                const float apq = m.a[pp][qq];
                if (fabsf(apq) < kTiny) {
                    continue;
                }
                const float theta = (m.a[qq][qq] - m.a[pp][pp]) / (2.f * apq);
                const float t = copysignf(1.f, theta) / (fabsf(theta) + sqrtf(theta * theta + 1.f));
                const float c = 1.f / sqrtf(t * t + 1.f), s = t * c;
                // A <- Jᵀ A J with J the rotation in the (p, q) plane
                for (int r = 0; r < 4; r++) {
                    const float rp = m.a[r][pp], rq = m.a[r][qq];
                    m.a[r][pp] = c * rp - s * rq, m.a[r][qq] = s * rp + c * rq;
                }
                for (int r = 0; r < 4; r++) {
                    const float pr = m.a[pp][r], qr = m.a[qq][r];
                    m.a[pp][r] = c * pr - s * qr, m.a[qq][r] = s * pr + c * qr;
                }
                for (int r = 0; r < 4; r++) {
                    const float rp = e[r][pp], rq = e[r][qq];
                    e[r][pp] = c * rp - s * rq, e[r][qq] = s * rp + c * rq;
                }
            }
        }
    }
    int top = 0;
    for (int i = 1; i < 4; i++) {
        top = m.a[i][i] > m.a[top][top] ? i : top;
    }
    for (int r = 0; r < 4; r++) {
        vec[r] = e[r][top];
    }
}
// The rotation that best maps the centred x onto the centred den in the weighted least-squares
// sense, by Horn's closed form (J. Opt. Soc. Am. A 4, 1987): with M = Σ w (x - x̄)(den - d̄)ᵀ, the unit
// quaternion of the rotation is the top eigenvector of the symmetric 4 x 4 matrix N(M).
struct Alignment {
    float rot[kXyz][kXyz]; // aligned = (x - x̄)·rot + d̄ for row vectors
    V3 x_mean, den_mean;
};
__device__ inline Alignment horn_alignment(const float (&mom)[kMoments]) {
    const float w = mom[0];
    float M[kXyz][kXyz];
    for (int a = 0; a < kXyz; a++) {
        for (int b = 0; b < kXyz; b++) {
            M[a][b] = mom[7 + 3 * a + b] - mom[1 + a] * mom[4 + b] / w;
        }
    }
    Sym4 n;
    const float diag[4] = {M[0][0] + M[1][1] + M[2][2], M[0][0] - M[1][1] - M[2][2], -M[0][0] + M[1][1] - M[2][2], -M[0][0] - M[1][1] + M[2][2]};
    const float skew[3] = {M[1][2] - M[2][1], M[2][0] - M[0][2], M[0][1] - M[1][0]};
    const float sym[3] = {M[0][1] + M[1][0], M[2][0] + M[0][2], M[1][2] + M[2][1]}; // (xy, zx, yz)
    for (int i = 0; i < 4; i++) {
        n.a[i][i] = diag[i];
    }
    for (int i = 0; i < 3; i++) {
        n.a[0][i + 1] = n.a[i + 1][0] = skew[i];
    }
    n.a[1][2] = n.a[2][1] = sym[0], n.a[1][3] = n.a[3][1] = sym[1], n.a[2][3] = n.a[3][2] = sym[2];
    float q[4];
    top_eigenvector(n, q);
    const float s = q[0], i = q[1], j = q[2], k = q[3];
    // the rotation matrix of the quaternion, acting on column vectors
    const float col[kXyz][kXyz] = {{s * s + i * i - j * j - k * k, 2 * (i * j - s * k), 2 * (i * k + s * j)},
                                   {2 * (i * j + s * k), s * s - i * i + j * j - k * k, 2 * (j * k - s * i)},
                                   {2 * (i * k - s * j), 2 * (j * k + s * i), s * s - i * i - j * j + k * k}};
    Alignment al;
    for (int a = 0; a < kXyz; a++) {
        for (int b = 0; b < kXyz; b++) {
            al.rot[a][b] = col[b][a]; // transposed: positions are row vectors here
        }
    }
    al.x_mean = V3{mom[1] / w, mom[2] / w, mom[3] / w};
    al.den_mean = V3{mom[4] / w, mom[5] / w, mom[6] / w};
    return al;
}
// REALIGN, second half: xn aligned rigidly onto den, then the Euler step from the aligned xn
// (reference: src/diffusion/positions.cuh:265-336). One thread solves the sample's alignment, the
// CTA's warps apply it to their tiles.
__device__ CCK_PHASE_FN void positions_realign(const KP& p, Deal& d, int step) {
    const int items = p.S * tile_groups(p);
    Alignment* shared = reinterpret_cast<Alignment*>(smem_base());
    const StepNoise sn = step_noise(p, step);
    const float dt = sn.sigma - sn.t_hat, scale = p.geo.misc[M_STEP_SCALE];
    for (int it = d.first(); it < items; it += gridDim.x) {
        const Tile t = group_tile(p, it);
        __syncthreads();
        if (threadIdx.x == 0) {
            float mom[kMoments];
            sample_sums(p.buf.kab, t.sample, p.chunks, mom);
            *shared = horn_alignment(mom);
        }
        __syncthreads();
        if (t.count == 0) {
            continue;
        }
        const Alignment& al = *shared;
        const V3 rel = tile_load(p.buf.xn, t) - al.x_mean, target = tile_load(p.buf.grad, t);
        const float means[kXyz] = {al.den_mean.x, al.den_mean.y, al.den_mean.z}, goal[kXyz] = {target.x, target.y, target.z};
        float out[kXyz];
#pragma unroll
        for (int a = 0; a < kXyz; a++) {
            const float moved = rel.x * al.rot[0][a] + rel.y * al.rot[1][a] + rel.z * al.rot[2][a] + means[a];
            out[a] = moved + scale * dt * (moved - goal[a]) / sn.t_hat;
        }
        tile_store(p.buf.pos, t, V3{out[0], out[1], out[2]});
    }
    __syncthreads();
    d.advance(items);
}

// ---- the atom input features: qa = ((xn·mask/√(t² + σd²)) @ WPOS (+ chirality gradient @ CHIR_W))·QMASK + SCQ

// CHIRAL: the gradient of (φ - ideal)² with respect to the atom in position `role` of the four that
// define the improper dihedral φ, by differentiating its construction backwards. Construction:
// b0 = p0 - p1, b1 = p2 - p1, b2 = p3 - p2, u = b1 / (|b1| + eps), v and w the parts of b0 and b2
// orthogonal to u, φ = atan2((u x v)·w + eps, v·w + eps)
// (reference: src/diffusion/positions.cuh:351-390).
__device__ __noinline__ V3 chiral_grad(const V3 (&pt)[4], float ideal, int role) {
    const V3 b0 = pt[0] - pt[1], b1 = pt[2] - pt[1], b2 = pt[3] - pt[2];
    const float len1 = sqrtf(dot(b1, b1)), den1 = len1 + kChiralEps;
    const V3 u = (1.f / den1) * b1;
    const float b0u = dot(b0, u), b2u = dot(b2, u);
    const V3 v = b0 - b0u * u, w = b2 - b2u * u;
    const V3 uxv = cross(u, v), wxu = cross(w, u), vxw = cross(v, w);
    const float y = dot(uxv, w) + kChiralEps, x = dot(v, w) + kChiralEps;
    // φ = atan2(y, x): dφ/dy = x / r², dφ/dx = -y / r²
    const float slope = 2.f * (atan2f(y, x) - ideal), r2 = x * x + y * y;
    const float dy = slope * x / r2, dx = -slope * y / r2;
    // y = (u x v)·w = (w x u)·v = (v x w)·u and x = v·w
    const V3 dv = dy * wxu + dx * w, dw = dy * uxv + dx * v;
    V3 du = dy * vxw;
    // v = b0 - (b0·u) u and w = b2 - (b2·u) u
    const float dvu = dot(dv, u), dwu = dot(dw, u);
    const V3 db0 = dv - dvu * u, db2 = dw - dwu * u;
    du = du - (dvu * b0 + b0u * dv + dwu * b2 + b2u * dw);
    // u = b1 / (|b1| + eps)
    const float dub1 = dot(du, b1);
    const V3 db1 = (1.f / den1) * du - (dub1 / (den1 * den1 * fmaxf(len1, 1e-30f))) * b1;
    // b0 = p0 - p1, b1 = p2 - p1, b2 = p3 - p2
    switch (role) {
    case 0:
        return db0;
    case 1:
        return -1.f * (db0 + db1);
    case 2:
        return db1 - db2;
    default:
        return db2;
    }
}
__device__ CCK_PHASE_FN void atom_init(const KP& p, Deal& d, float t) {
    const int rows = p.S * p.A;
    const float shrink = 1.f / sqrtf(t * t + kSigmaData * kSigmaData);
    const int col = 4 * lane_id();
    auto scaled_slot = [&](int sample, int slot) { // xn·mask/√(t² + σd²) of one slot
        const float* q = p.buf.xn + (size_t(sample) * nslots(p) + slot) * kXyz;
        const float w = p.geo.atom_mask[slot];
        return V3{q[0] * w * shrink, q[1] * w * shrink, q[2] * w * shrink};
    };
    for (int r = row_first(d); r < rows; r += row_step()) {
        const int sample = r / p.A, atom = r - sample * p.A, slot = p.geo.tok2q[atom];
        V3 x{0.f, 0.f, 0.f}, grad{0.f, 0.f, 0.f};
        if (slot >= 0) {
            x = scaled_slot(sample, slot);
            if (p.flags & F_CHIRAL) { // every chirality centre this slot takes part in (CSR: CHIR_PTR, CHIR_IDX = centre·4 + role)
                for (int edge = p.geo.chir_ptr[slot]; edge < p.geo.chir_ptr[slot + 1]; edge++) {
                    const int centre = p.geo.chir_idx[edge] >> 2, role = p.geo.chir_idx[edge] & 3;
                    const float ideal = p.geo.chir_a[centre];
                    if (ideal == 0.f) {
                        continue; // an angle of zero marks a centre to skip
                    }
                    V3 pt[4];
                    for (int k = 0; k < 4; k++) {
                        pt[k] = scaled_slot(sample, p.geo.chir_c[centre * 4 + k]);
                    }
                    const V3 g = chiral_grad(pt, ideal, role);
                    grad = grad + g;
                }
                grad = V3{isfinite(grad.x) ? grad.x : 0.f, isfinite(grad.y) ? grad.y : 0.f, isfinite(grad.z) ? grad.z : 0.f};
            }
        }
        const float xs[kXyz] = {x.x, x.y, x.z}, gs[kXyz] = {grad.x, grad.y, grad.z};
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int a = 0; a < kXyz; a++) {
            const float4 wp = ld4(p.geo.wpos + a * kAtomC + col);
            f = make_float4(f.x + xs[a] * wp.x, f.y + xs[a] * wp.y, f.z + xs[a] * wp.z, f.w + xs[a] * wp.w);
            if (p.flags & F_CHIRAL) {
                const float4 wc = ld4(p.geo.chir_w + a * kAtomC + col);
                f = make_float4(f.x + gs[a] * wc.x, f.y + gs[a] * wc.y, f.z + gs[a] * wc.z, f.w + gs[a] * wc.w);
            }
        }
        const float keep = p.geo.qmask[atom];
        const float4 base = ld4(p.geo.scq + size_t(atom) * kAtomC + col);
        *reinterpret_cast<float4*>(p.buf.qa + size_t(r) * kAtomC + col) =
            make_float4(f.x * keep + base.x, f.y * keep + base.y, f.z * keep + base.z, f.w * keep + base.w);
    }
    rows_done(d, rows);
}

// the operator's result: positions [S][Nb][24][3], zero past the real tokens; 128 bits per access
// (a token's 72 floats are 18 of them, so the real / padded boundary falls between two accesses)
__device__ CCK_PHASE_FN void positions_output(const KP& p, Deal& d) {
    if (!p.out) {
        return;
    }
    const int per = p.out_tokens * kSlots * kXyz / 4, real = nslots(p) * kXyz / 4, n = p.S * per, items = cdiv(n, kThreads);
    const float4* src = reinterpret_cast<const float4*>(p.buf.pos);
    float4* dst = reinterpret_cast<float4*>(p.out);
    for (int it = d.first(); it < items; it += gridDim.x) {
        const int i = it * kThreads + threadIdx.x;
        if (i < n) {
            const int sample = i / per, j = i - sample * per;
            dst[i] = j < real ? src[size_t(sample) * real + j] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    d.advance(items);
}

} // namespace cck

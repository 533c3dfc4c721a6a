// The token attention's inner loop on its own, in one CTA: two pipelines of four softmax warps (one
// thread per query row: S out of TMEM, scale + pair logits + maximum, exponentials, P into TMEM) and
// one MMA thread each (O += P.V from TMEM, S = Q.K two chunks ahead), handing over through the same
// mbarriers as the library's kernel, but with nothing else around it: operands sit in shared memory,
// no TMA, no other phase. Prints cycles per chunk of 64 keys and its split; what the library's kernel
// spends beyond this is the price of its surroundings.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o softmax_pipeline softmax_pipeline.cu -lcuda
//   ./softmax_pipeline
// VARIANT=1 (-DVARIANT=1): scalar fma/add instead of the packed f32x2 forms.
#include <cstdio>
#include <cstdlib>
#include "../csrc/ptx.cuh"
namespace cck { __device__ __forceinline__ long long wait_limit() { return 1ll << 31; } }
using namespace cck;
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
#ifndef VARIANT
#define VARIANT 0
#endif
constexpr int kChunks = 64;
__global__ void __launch_bounds__(384) body(long long* out, int sections, int mode) {
    extern __shared__ __align__(1024) char sm[];
    __shared__ uint32_t tmem_slot;
    __shared__ uint64_t mma_bar[2], s_full[2][2], p_full[2][2], pv_done[2][2];
    __shared__ volatile int stop, zero;
    __shared__ long long side[4];
    if (threadIdx.x == 0) {
        mbar_init(&mma_bar[0], 1), mbar_init(&mma_bar[1], 1);
        stop = 0, zero = 0;
        for (int a = 0; a < 2; a++) for (int c = 0; c < 2; c++) mbar_init(&s_full[a][c], 1), mbar_init(&p_full[a][c], 128), mbar_init(&pv_done[a][c], 1);
        fence_mbar_init();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    for (int i = threadIdx.x; i < 2 * 32768 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0x3f803f80u + i;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (warp >= 8) {
        const int r = warp - 8;
        if (lane == 0 && r < 2 && (r == 0 || !(mode & 16))) {
            const uint32_t tt = tmem + r * 256;
            const uint32_t idesc_s = umma_idesc_bf16(128, 64), idesc_o = umma_idesc_bf16(128, 48);
            const uint64_t dq = umma_desc_sw128(smem_u32(sm + 65536 + r * 32768)), dk = umma_desc_sw128(smem_u32(sm + 65536 + r * 32768 + 16384));
            auto qk = [&](int i) {
                for (int kk = 0; kk < 3; kk++) umma_bf16(tt + (i & 1) * 64, dq + 2 * kk, dk + 2 * kk, idesc_s, kk != 0);
                umma_commit(&s_full[r][i & 1]);
            };
            qk(0);
            qk(1);
            for (int i = 0; i < kChunks; i++) {
                const int bi = i & 1;
                mbar_wait(&p_full[r][bi], (i >> 1) & 1, (volatile int*)&stop);
                tc_fence_after();
                for (int kk = 0; kk < 4; kk++) umma_bf16_ts(tt + 192, tt + 128 + bi * 32 + 8 * kk, dk + 512 / 16 + 2 * kk, idesc_o, (i | kk) != 0);
                umma_commit(&pv_done[r][bi]);
                if (i + 2 < kChunks) qk(i + 2);
            }
            // everything issued is complete before TMEM goes away
            umma_commit(&mma_bar[r]);
            mbar_wait(&mma_bar[r], 0, (volatile int*)&stop);
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();
        __syncthreads();
        return;
    }
    const int t = warp >> 2, q = warp & 3, row_in = q * 32 + lane;
    const uint32_t tt = tmem + t * 256 + (uint32_t(q * 32) << 16);
    const float scale = 1.4426950408889634f / sqrtf(48.f);
    const float2 scale2 = make_float2(scale, scale);
    float m = 0.f, l = 0.f;
    long long tsec[4] = {0, 0, 0, 0}, twait = 0, twait2 = 0;
    if (t == 1 && (mode & 16)) { tc_fence_before(); __syncthreads(); __syncthreads(); return; }
    if (t == 1 && (mode & 32)) { const long long w0 = clock64(); while (clock64() - w0 < 700) {} }
    asm volatile("bar.sync %0, 128;" :: "r"(1 + t));
    const long long t0 = clock64();
    for (int g = 0; g < kChunks; g++) {
        const uint32_t bi = g & 1, bst = g & 1;
        long long cw = sections ? clock64() : 0;
        mbar_wait(&s_full[t][bi], (g >> 1) & 1, (volatile int*)&stop);
        tc_fence_after();
        long long c0 = sections ? clock64() : 0;
        twait += c0 - cw;
        uint32_t s0[32], s1[32];
        tmem_ld32_issue(tt + bi * 64, s0);
        tmem_ld32_issue(tt + bi * 64 + 32, s1);
        const char* brow = sm + t * 32768 + bst * 16384 + row_in * 128;
        tmem_ld_wait(s0);
        tmem_ld_wait(s1);
        long long c1 = sections ? clock64() : 0;
        float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        auto add_bias = [&](uint32_t(&sr)[32], int hf) {
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const uint4 bw = *reinterpret_cast<const uint4*>(brow + (((4 * hf + jj) ^ (row_in & 7)) << 4));
                const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int i = 8 * jj + 2 * k;
#if VARIANT == 0
                    const float2 a = __ffma2_rn(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), scale2,
                                                make_float2(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xFFFF0000u)));
#else
                    float2 a;
                    a.x = fmaf(__uint_as_float(sr[i]), scale, __uint_as_float(w[k] << 16));
                    a.y = fmaf(__uint_as_float(sr[i + 1]), scale, __uint_as_float(w[k] & 0xFFFF0000u));
#endif
                    sr[i] = __float_as_uint(a.x), sr[i + 1] = __float_as_uint(a.y);
                    mxp[k] = max3(mxp[k], a.x, a.y);
                }
            }
        };
        add_bias(s0, 0);
        add_bias(s1, 1);
#ifndef NOFENCE
        fence_async_smem();
#endif
        const float mx = max3(mxp[0], mxp[1], fmaxf(mxp[2], mxp[3]));
        long long c2 = sections ? clock64() : 0;
        if (g == 0) m = mx;
        else if (__any_sync(0xffffffffu, mx > m + 8.f)) { m = fmaxf(m, mx); l *= 0.5f; }
        long long cv = sections ? clock64() : 0;
        mbar_wait(&pv_done[t][bi], ((g >> 1) & 1) ^ 1, (volatile int*)&stop);
        long long cx = sections ? clock64() : 0;
        twait2 += cx - cv;
        const float2 neg_m = make_float2(-m, -m);
        float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        auto exp_store = [&](const uint32_t(&sr)[32], int hf) {
#pragma unroll
            for (int jj = 0; jj < 2; jj++) {
                uint32_t pk[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
#if VARIANT == 0
                    const float2 x = __fadd2_rn(make_float2(__uint_as_float(sr[16 * jj + 2 * k]), __uint_as_float(sr[16 * jj + 2 * k + 1])), neg_m);
                    const float2 e = make_float2(ex2_fast(x.x), ex2_fast(x.y));
                    sum2[k & 1] = __fadd2_rn(sum2[k & 1], e);
#else
                    float2 e;
                    e.x = ex2_fast(__uint_as_float(sr[16 * jj + 2 * k]) - m);
                    e.y = ex2_fast(__uint_as_float(sr[16 * jj + 2 * k + 1]) - m);
                    sum2[k & 1].x += e.x, sum2[k & 1].y += e.y;
#endif
                    pk[k] = pack_bf2(e.x, e.y);
                }
                tmem_st8(tt + 128 + bi * 32 + 16 * hf + 8 * jj, pk);
            }
        };
        exp_store(s0, 0);
        exp_store(s1, 1);
        l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        long long c3 = sections ? clock64() : 0;
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[t][bi]);
        long long c4 = sections ? clock64() : 0;
        tsec[0] += c1 - c0, tsec[1] += c2 - c1, tsec[2] += c3 - c2, tsec[3] += c4 - c3;
    }
    const long long t1 = clock64();
    if (threadIdx.x == 0) side[0] = twait, side[1] = twait2;
    if (l == 123.456f) out[63] = 1;
    if (threadIdx.x == 0) {
        out[0] = t1 - t0;
        for (int i = 0; i < 4; i++) out[1 + i] = tsec[i];
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) for (int i = 0; i < 4; i++) out[5 + i] = side[i];
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
int main(int argc, char** argv) {
    const int threads = argc > 1 ? atoi(argv[1]) : 384;
    long long* d;
    cudaMalloc(&d, 512);
    const int smem = 131072 + 1024;
    cudaFuncSetAttribute(body, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int modes[] = {0, 16, 32};
    for (int mode : modes) {
        long long h[9];
        body<<<1, threads, smem>>>(d, 1, mode);
        body<<<1, threads, smem>>>(d, 1, mode);
        cudaDeviceSynchronize();
        cudaMemcpy(h, d, 72, cudaMemcpyDeviceToHost);
        printf("mode %2d (0 both pipelines, 16 one pipeline, 32 second pipeline starts 700 cycles late): %7.1f cycles per chunk [S ld %6.1f | bias+max %6.1f | exp+P %6.1f | st wait %5.1f]  waits S %lld P-buffer %lld per chunk (%lld %lld)\n",
               mode, double(h[0]) / kChunks, double(h[1]) / kChunks, double(h[2]) / kChunks, double(h[3]) / kChunks, double(h[4]) / kChunks, h[5] / kChunks, h[6] / kChunks, h[7], h[8]);
    }
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

// Plain global stores of 120 CTAs at once, each writing its own 128 x 128 f32 tile of a [2560][768]
// matrix from eight warps: bytes per clock per SM for three footprints of a warp's store instruction
// (0: 8 rows x 64 bytes, the gated-residual epilogue's; 1: one row x 512 bytes; 2: 32 rows x 16 bytes, a
// thread per row), with little and with 200 KB of dynamic shared memory.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o store_rates store_rates.cu
//   ./store_rates
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__global__ void __launch_bounds__(384, 1) st(float* out, long long* cyc, int pattern, int reps, size_t ld) {
    extern __shared__ char sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // each CTA owns a tile of 128 rows x 128 floats (row pitch ld floats), rewritten reps times
    float* tile = out + size_t(blockIdx.x % 20) * 128 * ld + (blockIdx.x / 20) * 128;
    const float4 v = make_float4(lane, warp, 1.f, 2.f);
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < reps && warp < 8; r++) {
        if (pattern == 0) {        // 8 rows x 64 B per instruction (4 lanes per row): the gated-residual epilogue's
            const int q = warp & 3, g = warp >> 2;
            for (int k = 0; k < 4; k++)
                for (int i = 0; i < 4; i++) {
                    const int row = q * 32 + (lane >> 2) + 8 * i, col = g * 64 + k * 16 + 4 * (lane & 3);
                    *reinterpret_cast<float4*>(tile + size_t(row) * ld + col) = v;
                }
        } else if (pattern == 1) { // 1 row x 512 B per instruction
            for (int k = 0; k < 16; k++) {
                const int row = warp * 16 + k;
                *reinterpret_cast<float4*>(tile + size_t(row) * ld + 4 * lane) = v;
            }
        } else if (pattern == 2) { // 32 rows x 16 B per instruction (a thread per row)
            const int q = warp & 3, g = warp >> 2;
            for (int k = 0; k < 16; k++) {
                const int row = q * 32 + lane, col = g * 64 + 4 * k;
                *reinterpret_cast<float4*>(tile + size_t(row) * ld + col) = v;
            }
        }
    }
    const long long t1 = clock64();
    __syncthreads();
    if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
    if (sm[threadIdx.x & 255] == 77) cyc[147] = 0;
}
int main() {
    float* out; long long* cyc;
    const size_t ld = 768;
    cudaMalloc(&out, size_t(2560) * ld * 4 * 2);
    cudaMalloc(&cyc, 148 * 8);
    for (int smem : {1024, 200 * 1024}) {
        cudaFuncSetAttribute(st, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        for (int pattern = 0; pattern < 3; pattern++)
            for (int reps : {1, 8}) {
                st<<<120, 384, smem>>>(out, cyc, pattern, reps, ld);
                st<<<120, 384, smem>>>(out, cyc, pattern, reps, ld);
                cudaDeviceSynchronize();
                long long h[148];
                cudaMemcpy(h, cyc, 120 * 8, cudaMemcpyDeviceToHost);
                double s = 0; long long mx = 0;
                for (int i = 0; i < 120; i++) { s += h[i]; if (h[i] > mx) mx = h[i]; }
                printf("smem %3d KB pattern %d reps %d: %8.0f cycles avg, %8lld max per CTA: %.1f B/clk/SM\n", smem / 1024, pattern, reps, s / 120, mx, 65536.0 * reps / (s / 120));
            }
    }
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
}

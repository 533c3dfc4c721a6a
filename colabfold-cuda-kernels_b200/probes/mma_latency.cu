// Latencies of the tensor-core pipelines' building blocks, one CTA: a batch of tcgen05.mma -> commit ->
// the issuing thread sees the mbarrier complete (per batch size and shape, so that the difference
// between two sizes is the cost of an MMA), and 128 threads <-> 1 thread through two mbarriers.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o mma_latency mma_latency.cu -lcuda
//   ./mma_latency
#include <cstdio>
#include <cstdlib>
#include "../csrc/ptx.cuh"
namespace cck { __device__ __forceinline__ long long wait_limit() { return 1ll << 28; } }
using namespace cck;
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
constexpr int kTurns = 200;
__global__ void __launch_bounds__(256) lat(long long* out, int nqk, int npv, int nq_n, int pingpong) {
    extern __shared__ __align__(1024) char sm[];
    __shared__ uint32_t tmem_slot;
    __shared__ uint64_t bar, ping, pong;
    __shared__ volatile int stop;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    if (threadIdx.x == 0) { mbar_init(&bar, 1), mbar_init(&ping, 128), mbar_init(&pong, 1); stop = 0; fence_mbar_init(); }
    for (int i = threadIdx.x; i < 65536 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0x3c003c00u;
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (!pingpong) {
        if (threadIdx.x == 0) {
            const uint32_t idesc_s = umma_idesc_bf16(128, nq_n), idesc_o = umma_idesc_bf16(128, 48);
            const uint64_t dq = umma_desc_sw128(smem_u32(sm)), dk = umma_desc_sw128(smem_u32(sm + 16384));
            uint32_t par = 0;
            const long long t0 = clock64();
            for (int n = 0; n < kTurns; n++) {
                for (int kk = 0; kk < nqk; kk++) umma_bf16(tmem + (n & 1) * 64, dq + 2 * (kk % 3), dk + 2 * (kk % 3), idesc_s, kk != 0);
                for (int kk = 0; kk < npv; kk++) umma_bf16_ts(tmem + 192, tmem + 128 + 8 * (kk % 4), dk + 2 * (kk % 4), idesc_o, 1);
                umma_commit(&bar);
                mbar_wait(&bar, par, &stop);
                par ^= 1;
            }
            out[0] = clock64() - t0;
        }
    } else {
        // 128 threads arrive on ping; one thread (warp 4 lane 0) waits, arrives on pong; the 128 wait for pong
        if (warp < 4) {
            const long long t0 = clock64();
            for (int n = 0; n < kTurns; n++) {
                mbar_arrive(&ping);
                mbar_wait(&pong, n & 1, &stop);
            }
            if (threadIdx.x == 0) out[0] = clock64() - t0;
        } else if (warp == 4 && lane == 0) {
            for (int n = 0; n < kTurns; n++) {
                mbar_wait(&ping, n & 1, &stop);
                mbar_arrive(&pong);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
    long long* d;
    cudaMalloc(&d, 512);
    cudaFuncSetAttribute(lat, cudaFuncAttributeMaxDynamicSharedMemorySize, 66560);
    auto run = [&](const char* what, int nqk, int npv, int nq_n, int pp) {
        long long h = 0;
        lat<<<1, 256, 66560>>>(d, nqk, npv, nq_n, pp);
        lat<<<1, 256, 66560>>>(d, nqk, npv, nq_n, pp);
        cudaDeviceSynchronize();
        cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
        printf("%-58s %7.1f cycles per turn\n", what, double(h) / kTurns);
    };
    run("commit only -> wait", 0, 0, 64, 0);
    run("1 QK MMA (128x64x16) -> commit -> wait", 1, 0, 64, 0);
    run("3 QK MMA (128x64x16) -> commit -> wait", 3, 0, 64, 0);
    run("6 QK MMA", 6, 0, 64, 0);
    run("12 QK MMA", 12, 0, 64, 0);
    run("24 QK MMA", 24, 0, 64, 0);
    run("24 QK MMA with N=128", 24, 0, 128, 0);
    run("24 QK MMA with N=256", 24, 0, 256, 0);
    run("4 PV MMA (TS 128x48x16)", 0, 4, 64, 0);
    run("8 PV MMA", 0, 8, 64, 0);
    run("16 PV MMA", 0, 16, 64, 0);
    run("32 PV MMA", 0, 32, 64, 0);
    run("3 QK + 4 PV (one chunk)", 3, 4, 64, 0);
    run("ping-pong 128 threads <-> 1 thread through mbarriers", 0, 0, 64, 1);
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

// Throughput of single instructions on one SM sub-partition: W warps per sub-partition (W = 1, 2), each
// issuing 512 independent instances of one instruction kind over 8 register chains; cycles per
// warp-instruction. (Forms that the compiler folds away print 0.)
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o instruction_rates instruction_rates.cu
//   ./instruction_rates
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

#define OPS 512
template <int KIND> __device__ __forceinline__ void op(uint32_t (&r)[8], int i) {
    uint32_t& a = r[i & 7];
    const uint32_t b = r[(i + 3) & 7];
    if (KIND == 0) asm volatile("shl.b32 %0, %0, 1;" : "+r"(a));
    if (KIND == 1) asm volatile("and.b32 %0, %0, %1;" : "+r"(a) : "r"(0xffff0001u | i));
    if (KIND == 2) asm volatile("max.f32 %0, %0, %1;" : "+r"(a) : "r"(b));
    if (KIND == 3) asm volatile("max.f32 %0, %0, %1, %2;" : "+r"(a) : "r"(b), "r"(r[(i + 5) & 7]));
    if (KIND == 4) asm volatile("cvt.rn.bf16x2.f32 %0, %0, %1;" : "+r"(a) : "r"(b));
    if (KIND == 5) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+r"(a));
    if (KIND == 6) asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+r"(a) : "r"(b));
    if (KIND == 7) asm volatile("add.f32 %0, %0, %1;" : "+r"(a) : "r"(b));
    if (KIND == 8) asm volatile("prmt.b32 %0, %0, %1, 0x5410;" : "+r"(a) : "r"(b));
    if (KIND == 9) asm volatile("mul.lo.u32 %0, %0, 65536;" : "+r"(a));
    if (KIND == 10) asm volatile("mad.lo.u32 %0, %0, 65536, %1;" : "+r"(a) : "r"(b));
    if (KIND == 11) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(a) : "r"(b), "r"(r[(i + 5) & 7]));
    if (KIND == 12) asm volatile("shf.l.wrap.b32 %0, %0, %1, 16;" : "+r"(a) : "r"(b));
    if (KIND == 13) asm volatile("sub.f32 %0, %0, %1;" : "+r"(a) : "r"(b));
}
template <int KIND> __device__ __forceinline__ void op2(unsigned long long (&r)[8], int i) {
    unsigned long long& a = r[i & 7];
    const unsigned long long b = r[(i + 3) & 7];
    if (KIND == 20) asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(a) : "l"(b));
    if (KIND == 21) asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(a) : "l"(b));
}
template <int KIND> __global__ void bench(long long* out, uint32_t seed) {
    uint32_t r[8];
    unsigned long long q[8];
    for (int i = 0; i < 8; i++) {
        r[i] = seed * (threadIdx.x + 1) + i * 0x3f800000u, q[i] = (unsigned long long)(r[i]) << 32 | 0x3f800000u;
    }
    __syncthreads();
    const long long t0 = clock64();
#pragma unroll
    for (int i = 0; i < OPS; i++) {
        if (KIND < 20) op<KIND>(r, i);
        else op2<KIND>(q, i);
    }
    const long long t1 = clock64();
    uint32_t acc = 0;
    for (int i = 0; i < 8; i++) acc ^= r[i] ^ uint32_t(q[i]) ^ uint32_t(q[i] >> 32);
    if (acc == 0x12345678u) out[63] = acc;
    if (threadIdx.x == 0) out[0] = t1 - t0;
}
template <int KIND> void run(const char* name, long long* d) {
    for (int warps = 4; warps <= 8; warps += 4) { // 4 warps = 1 per SMSP, 8 = 2 per SMSP
        long long h = 0;
        bench<KIND><<<1, 32 * warps>>>(d, 12345);
        bench<KIND><<<1, 32 * warps>>>(d, 12345);
        cudaDeviceSynchronize();
        cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
        printf("%-28s %d warp(s)/SMSP: %6.2f cycles per warp-instruction\n", name, warps / 4, double(h) / OPS);
    }
}
int main() {
    long long* d;
    cudaMalloc(&d, 512);
    run<0>("shl.b32", d); run<12>("shf.l.wrap", d); run<1>("and.b32", d); run<11>("lop3", d); run<8>("prmt", d);
    run<9>("mul.lo.u32 (x65536)", d); run<10>("mad.lo.u32", d);
    run<2>("max.f32 (2 in)", d); run<3>("max.f32 (3 in)", d);
    run<4>("cvt.rn.bf16x2.f32", d); run<5>("ex2.approx.ftz.f32", d);
    run<6>("fma.rn.f32", d); run<7>("add.f32", d); run<13>("sub.f32", d);
    run<20>("fma.rn.f32x2", d); run<21>("add.rn.f32x2", d);
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

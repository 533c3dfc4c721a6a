// Test infrastructure, not product code: NVIDIA's own Philox4x32-10 (the cuRAND device header,
// which also compiles for the host) behind a C entry point, as an independent implementation to
// hold the sampler's and the oracle's raw Philox words against. Only tests load this library.
#include <cstdint>

#include <vector_types.h>
#define QUALIFIERS static inline
#include <curand_philox4x32_x.h>

extern "C" void kat_curand_philox(const uint32_t* counter, const uint32_t* key, uint32_t* out) {
    const uint4 c = {counter[0], counter[1], counter[2], counter[3]};
    const uint2 k = {key[0], key[1]};
    const uint4 r = curand_Philox4x32_10(c, k);
    out[0] = r.x, out[1] = r.y, out[2] = r.z, out[3] = r.w;
}

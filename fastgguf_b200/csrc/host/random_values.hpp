// The seeded generator of random weights, as one function that the host and the device both compile:
// integer arithmetic, one integer-to-float conversion and individually rounded float operations, so that a
// model folder written on the CPU and weights generated on the GPU from the same seed hold the same bits.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define FG_HD __host__ __device__ __forceinline__
#else
#define FG_HD inline
#endif

namespace fg {

FG_HD uint64_t mix64(uint64_t z) {            // the splitmix64 finaliser
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ~ N(0, 1): the sum of eight uniform 24-bit integers, centred, times 1 / (2^24 * sqrt(8 / 12)).
FG_HD float random_unit_normal(uint64_t seed, uint64_t name_hash, uint64_t index) {
    uint64_t base = mix64(seed + 0x9E3779B97F4A7C15ull * (index + 1)) ^ name_hash;
    int64_t sum = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int k = 0; k < 4; k++) {
        uint64_t w = mix64(base + 0xD1B54A32D192ED03ull * (uint64_t)(k + 1));
        sum += (int64_t)(w & 0xFFFFFFull) + (int64_t)((w >> 24) & 0xFFFFFFull);
    }
    sum -= 4 * 0xFFFFFFll;
    const float scale = 7.3001261e-8f;        // 1 / (16777216 * 0.81649658)
#if defined(__CUDA_ARCH__)
    return __fmul_rn((float)sum, scale);
#else
    volatile float v = (float)sum * scale;
    return v;
#endif
}

// init 0: std * z; init 1: 1 + std * z (each operation rounded on its own, no fused multiply-add)
FG_HD float random_weight(uint64_t seed, uint64_t name_hash, uint64_t index, int init, float std) {
    float z = random_unit_normal(seed, name_hash, index);
#if defined(__CUDA_ARCH__)
    float v = __fmul_rn(z, std);
    return init == 1 ? __fadd_rn(1.0f, v) : v;
#else
    volatile float v = z * std;
    if (init == 1) { volatile float w = 1.0f + v; return w; }
    return v;
#endif
}

FG_HD uint16_t bf16_bits_rne(float f) {
    union { float f; uint32_t u; } c;
    c.f = f;
    uint32_t u = c.u;
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040u);   // NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

}  // namespace fg

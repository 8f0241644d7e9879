// anvil_rng.h — the counter-based random numbers shared by host code and kernels.
//
// Restates anvil/backend/anvil_host.h:17-29 (and anvil/interp.py:55-71): 32 bits per
// (element index, stream, salt, seed), two rounds of the lowbias32 integer hash; a uniform float
// is the top 24 bits scaled by 2^-24, in [0, 1), or in (0, 1] when open_low is set.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ANVIL_HD __host__ __device__ __forceinline__
#else
#define ANVIL_HD static inline
#endif

ANVIL_HD uint32_t anvil_lowbias32(uint32_t x) {
    x ^= x >> 16; x *= 0x7FEB352Du;
    x ^= x >> 15; x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}

ANVIL_HD uint32_t anvil_rand_bits(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed) {
    uint32_t k = stream * 0x85EBCA77u + salt * 0xC2B2AE3Du + seed + 0x632BE5ABu;
    return anvil_lowbias32(anvil_lowbias32(idx * 0x9E3779B1u + k));
}

// (bits >> 8) [+ 1] is at most 2^24, exactly representable in f32, and the scale is a power of two,
// so the f32 product equals the reference's double computation rounded to f32.
ANVIL_HD float anvil_rand(uint32_t idx, uint32_t stream, uint32_t salt, uint32_t seed, int open_low) {
    uint32_t hi = (anvil_rand_bits(idx, stream, salt, seed) >> 8) + (open_low ? 1u : 0u);
    return (float)hi * (1.0f / 16777216.0f);
}

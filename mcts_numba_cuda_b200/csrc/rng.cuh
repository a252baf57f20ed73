// xoroshiro128+ streams, bit-compatible with numba.cuda.random (third party; numba 0.65.0), which the reference
// uses for every random draw (call sites src/mctsnc.py:391-394,1435,1511,1882,1971,2061).  Restated from the
// published algorithm: SplitMix64 seeding, rotations 55/14/36, the 2^64 jump polynomial, and the conversion
// float32(float64(x >> 11) * 2^-53), which can round up to exactly 1.0f.
#pragma once


#if defined(__CUDACC__)
#define MCTS_HD __host__ __device__ __forceinline__
#else
#define MCTS_HD inline
#endif

namespace mctsnc {

struct RngState {
    unsigned long long s0, s1;
};

MCTS_HD unsigned long long rotl64(unsigned long long x, int k) { return (x << k) | (x >> (64 - k)); }

MCTS_HD unsigned long long rng_next(unsigned long long &s0, unsigned long long &s1) {
    unsigned long long result = s0 + s1;
    s1 ^= s0;
    s0 = rotl64(s0, 55) ^ s1 ^ (s1 << 14);
    s1 = rotl64(s1, 36);
    return result;
}

inline void rng_seed(RngState &s, unsigned long long seed) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    s.s0 = z;
    s.s1 = z;
}

inline void rng_jump(RngState &s) {
    const unsigned long long jump[2] = {0xbeac0467eba5facbULL, 0xd86b048b86aa9922ULL};
    unsigned long long a = 0, b = 0;
    for (int i = 0; i < 2; i++)
        for (int bit = 0; bit < 64; bit++) {
            if (jump[i] & (1ULL << bit)) {
                a ^= s.s0;
                b ^= s.s1;
            }
            rng_next(s.s0, s.s1);
        }
    s.s0 = a;
    s.s1 = b;
}

#if defined(__CUDACC__)
// uniform float32 of numba: the 53-bit integer x >> 11 is exact in float64, so one round-to-nearest conversion of the
// integer to float32 followed by the exact scaling 2^-53 gives the same value as float32(float64(v) * 2^-53).
__device__ __forceinline__ float rng_uniform_f32(unsigned long long &s0, unsigned long long &s1) {
    unsigned long long x = rng_next(s0, s1);
    return __fmul_rn(__ull2float_rn(x >> 11), 1.1102230246251565e-16f);
}

// The same uniform scaled by 2^64, for callers that fold the scaling into a constant of their own: clearing the low 11
// bits instead of shifting them out gives (x >> 11) * 2^11, whose conversion rounds exactly like that of x >> 11
// (a power-of-two factor moves no rounding boundary, and 2^64 is representable), so
// rng_uniform_f32() == rng_uniform_times_2p64() * 2^-64 bit for bit; the value 2^64 stands for 1.0f.
constexpr float RNG_2P64 = 18446744073709551616.f;
constexpr float RNG_2M64 = 5.421010862427522e-20f;
__device__ __forceinline__ float rng_uniform_times_2p64(unsigned long long &s0, unsigned long long &s1) {
    return __ull2float_rn(rng_next(s0, s1) & ~0x7FFULL);
}
#endif

}  // namespace mctsnc

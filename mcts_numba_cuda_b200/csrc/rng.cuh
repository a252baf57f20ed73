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

// ---------------------------------------------------------------------------------------------------------------
// Stream i of create_xoroshiro128p_states is the seeded state jumped i times by 2^64 steps
// (numba/cuda/random.py:226-243: a sequential chain on the host).  The state update and therefore the jump are linear
// over GF(2), so "jump 2^k times" is a 128 x 128 bit matrix J^(2^k), and stream i is the product of the matrices of the set
// bits of i applied to the seeded state: every stream can be computed on its own, in at most JUMP_LEVELS matrix-vector
// products, on the device.  A matrix is stored by columns (column c = image of the state with only bit c set; bits 0..63
// are s0, bits 64..127 are s1), so a product is the XOR of the columns selected by the set bits of the state.
constexpr int JUMP_LEVELS = 28;   // stream indices below 2^28 (512 trees x 512 actions x 512 playouts = 2^27)

struct JumpColumn {
    unsigned long long s0, s1;
};

MCTS_HD void jump_apply(const JumpColumn *cols, unsigned long long &s0, unsigned long long &s1) {
    unsigned long long a0 = 0, a1 = 0;
    for (int c = 0; c < 64; c++) {
        const unsigned long long m0 = 0ULL - ((s0 >> c) & 1ULL), m1 = 0ULL - ((s1 >> c) & 1ULL);
        a0 ^= (cols[c].s0 & m0) ^ (cols[64 + c].s0 & m1);
        a1 ^= (cols[c].s1 & m0) ^ (cols[64 + c].s1 & m1);
    }
    s0 = a0;
    s1 = a1;
}

// fills cols[JUMP_LEVELS][128]: level 0 from rng_jump on the 128 unit states, level k+1 = level k applied to itself
inline void jump_matrices(JumpColumn *cols) {
    for (int c = 0; c < 128; c++) {
        RngState s;
        s.s0 = c < 64 ? 1ULL << c : 0ULL;
        s.s1 = c < 64 ? 0ULL : 1ULL << (c - 64);
        rng_jump(s);
        cols[c].s0 = s.s0;
        cols[c].s1 = s.s1;
    }
    for (int k = 1; k < JUMP_LEVELS; k++)
        for (int c = 0; c < 128; c++) {
            unsigned long long s0 = cols[(k - 1) * 128 + c].s0, s1 = cols[(k - 1) * 128 + c].s1;
            jump_apply(cols + (k - 1) * 128, s0, s1);
            cols[k * 128 + c].s0 = s0;
            cols[k * 128 + c].s1 = s1;
        }
}

#if defined(__CUDACC__)
// out[i] = stream first + i * stride of create_xoroshiro128p_states(*, seed): (seed0, seed1) is the seeded state
__global__ void init_streams_kernel(ulonglong2 *out, const JumpColumn *cols, unsigned long long seed0, unsigned long long seed1,
                                    long long first, long long stride, long long count) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long index = (unsigned long long)(first + i * stride);
        unsigned long long s0 = seed0, s1 = seed1;
        for (int k = 0; k < JUMP_LEVELS; k++)
            if ((index >> k) & 1ULL) jump_apply(cols + k * 128, s0, s1);
        out[i] = make_ulonglong2(s0, s1);
    }
}

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

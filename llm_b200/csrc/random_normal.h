// A counter-based normal generator that gives the same bits on the host, on the device and
// in the plain numpy statement of the tests: element i of a tensor depends only on
// (key, i), where the key is made from the seed and the tensor's name. It plays the part of
// the seeded fixture writer of MythEclipse/llm (scripts/make_tiny_moe.py:93-119), which draws
// its matrices from one seeded generator; here no order of drawing exists at all.
//
//   x      = splitmix64 finalizer of (key + (i + 1) * 0x9E3779B97F4A7C15)
//   u1     = ((x >> 40) + 1) / 2^24                in (0, 1]
//   theta  = (((x >> 16) & 0x3FFFFF) + 0.5) / 2^22 * (pi / 2), quadrant = (x >> 38) & 3
//   z      = sqrt(-2 ln u1) * cos(theta + quadrant * pi / 2)            (Box-Muller)
//
// ln, cos and sin are written out here with additions, multiplications and divisions only
// (an atanh series and Taylor polynomials), each a single correctly rounded 32-bit operation:
// no fused multiply-add, no library function whose rounding differs between machines. The
// host library is compiled with -ffp-contract=off, device code uses the _rn intrinsics.
#pragma once

#include <cstdint>

#if defined(__CUDA_ARCH__)
#define LLMB_RN_HD __host__ __device__ __forceinline__
#define LLMB_MUL(a, b) __fmul_rn((a), (b))
#define LLMB_ADD(a, b) __fadd_rn((a), (b))
#define LLMB_DIV(a, b) __fdiv_rn((a), (b))
#define LLMB_SQRT(a) __fsqrt_rn((a))
#elif defined(__CUDACC__)
#include <cmath>
#define LLMB_RN_HD __host__ __device__ inline
#define LLMB_MUL(a, b) ((a) * (b))
#define LLMB_ADD(a, b) ((a) + (b))
#define LLMB_DIV(a, b) ((a) / (b))
#define LLMB_SQRT(a) sqrtf((a))
#else
#include <cmath>
#define LLMB_RN_HD inline
#define LLMB_MUL(a, b) ((a) * (b))
#define LLMB_ADD(a, b) ((a) + (b))
#define LLMB_DIV(a, b) ((a) / (b))
#define LLMB_SQRT(a) std::sqrt((a))
#endif

namespace llmb_random {

LLMB_RN_HD uint64_t mix(uint64_t key, uint64_t index) {
    uint64_t x = key + (index + 1ull) * 0x9E3779B97F4A7C15ull;
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

// ln(u) for u = a / 2^24, 1 <= a <= 2^24: u = m * 2^e with 1 <= m < 2;
// ln m = 2 s (1 + s^2/3 + s^4/5 + ... + s^12/13), s = (m - 1) / (m + 1)
LLMB_RN_HD float log_unit(uint32_t a) {
    int shift = 0;
    while ((a << shift) < (1u << 24)) ++shift;        // a << shift in [2^24, 2^25)
    float m = LLMB_MUL((float)(a << shift), 5.9604644775390625e-08f);      // * 2^-24: in [1, 2)
    float e = (float)(-shift);
    float s = LLMB_DIV(LLMB_ADD(m, -1.0f), LLMB_ADD(m, 1.0f));
    float s2 = LLMB_MUL(s, s);
    float p = 1.0f / 13.0f;
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f / 11.0f);
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f / 9.0f);
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f / 7.0f);
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f / 5.0f);
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f / 3.0f);
    p = LLMB_ADD(LLMB_MUL(p, s2), 1.0f);
    float ln_m = LLMB_MUL(LLMB_MUL(2.0f, s), p);
    return LLMB_ADD(LLMB_MUL(e, 0.693147182464599609375f), ln_m);
}

// cos and sin of t in (0, pi/2) by their Taylor polynomials in t^2
LLMB_RN_HD void cos_sin(float t, float& c, float& s) {
    float t2 = LLMB_MUL(t, t);
    float pc = -1.0f / 87178291200.0f;                                  // -1/14!
    pc = LLMB_ADD(LLMB_MUL(pc, t2), 1.0f / 479001600.0f);               // 1/12!
    pc = LLMB_ADD(LLMB_MUL(pc, t2), -1.0f / 3628800.0f);
    pc = LLMB_ADD(LLMB_MUL(pc, t2), 1.0f / 40320.0f);
    pc = LLMB_ADD(LLMB_MUL(pc, t2), -1.0f / 720.0f);
    pc = LLMB_ADD(LLMB_MUL(pc, t2), 1.0f / 24.0f);
    pc = LLMB_ADD(LLMB_MUL(pc, t2), -0.5f);
    c = LLMB_ADD(LLMB_MUL(pc, t2), 1.0f);
    float ps = 1.0f / 6227020800.0f;                                    // 1/13!
    ps = LLMB_ADD(LLMB_MUL(ps, t2), -1.0f / 39916800.0f);
    ps = LLMB_ADD(LLMB_MUL(ps, t2), 1.0f / 362880.0f);
    ps = LLMB_ADD(LLMB_MUL(ps, t2), -1.0f / 5040.0f);
    ps = LLMB_ADD(LLMB_MUL(ps, t2), 1.0f / 120.0f);
    ps = LLMB_ADD(LLMB_MUL(ps, t2), -1.0f / 6.0f);
    ps = LLMB_ADD(LLMB_MUL(ps, t2), 1.0f);
    s = LLMB_MUL(ps, t);
}

// One standard normal value for (key, index).
LLMB_RN_HD float standard_normal(uint64_t key, uint64_t index) {
    uint64_t x = mix(key, index);
    uint32_t a = (uint32_t)(x >> 40) + 1u;                              // 1 .. 2^24
    uint32_t quadrant = (uint32_t)(x >> 38) & 3u;
    uint32_t b = (uint32_t)(x >> 16) & 0x3FFFFFu;                       // 22 bits
    float radius = LLMB_SQRT(LLMB_MUL(-2.0f, log_unit(a)));
    float t = LLMB_MUL(LLMB_MUL(LLMB_ADD((float)b, 0.5f), 2.384185791015625e-07f),      // / 2^22
                       1.57079637050628662109375f);                                      // * pi/2
    float c, s;
    cos_sin(t, c, s);
    float direction = quadrant == 0 ? c : quadrant == 1 ? -s : quadrant == 2 ? -c : s;
    return LLMB_MUL(radius, direction);
}

// mean + deviation * z, rounded once more to bfloat16 (nearest even) where asked
LLMB_RN_HD float value(uint64_t key, uint64_t index, float mean, float deviation) {
    return LLMB_ADD(mean, LLMB_MUL(deviation, standard_normal(key, index)));
}

LLMB_RN_HD uint16_t to_bfloat16_bits(float v) {
    union { float f; uint32_t u; } w;
    w.f = v;
    uint32_t u = w.u;
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x40u);   // NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

}  // namespace llmb_random

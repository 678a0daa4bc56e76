/* r3d_numerics.cuh -- the scalar number formats of the quantised-matmul path, usable from
 * host and device code. Every function is bit-exact to the rule libr3d states at the cited
 * line; the kernels' faster packed converters are tested against these.
 */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#define R3D_HD __host__ __device__ __forceinline__

namespace r3d {

R3D_HD float bits_f32(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    union { uint32_t u; float f; } v; v.u = u; return v.f;
#endif
}
R3D_HD uint32_t f32_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    union { uint32_t u; float f; } v; v.f = f; return v.u;
#endif
}

/* bf16: widening is a shift; narrowing rounds to nearest even and quiets NaN
 * (src/r3d_gemm_fp8a8.hip:101-105). */
R3D_HD float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
R3D_HD uint16_t f32_to_bf16(float f) {
    const uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

/* IEEE binary16 -> f32, exact (scale planes of the LM head may be f16,
 * src/r3d_gemm_logits.hip:65-69). */
R3D_HD float f16_to_f32(uint16_t h) {
    const uint32_t s = (uint32_t)(h >> 15) << 31;
    const uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0u) {
        if (m == 0u) return bits_f32(s);
        const float f = (float)m * 5.9604644775390625e-08f;   /* m * 2^-24, exact */
        return bits_f32(s | f32_bits(f));
    }
    if (e == 31u) return bits_f32(s | 0x7f800000u | (m << 13));
    return bits_f32(s | ((e + 112u) << 23) | (m << 13));
}

/* e4m3fn -> f32 (src/r3d_gemm_fp8a8.hip:134-150): bias 7, no infinities, S.1111.111 is the
 * only NaN, subnormals are m * 2^-9, the sign of zero is kept. */
R3D_HD float e4m3_to_f32(uint8_t b) {
    const uint32_t s = (uint32_t)(b >> 7) << 31;
    const uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
    if (e == 0u) {
        if (m == 0u) return bits_f32(s);
        const float f = (float)m * 0.001953125f;              /* m * 2^-9, exact */
        return bits_f32(s | f32_bits(f));
    }
    if (e == 0xfu && m == 7u) return bits_f32(s | 0x7fc00000u);
    return bits_f32(s | ((e + 120u) << 23) | (m << 20));
}

/* f32 -> e4m3fn, round to nearest even, saturating at +-448, NaN -> S.1111.111
 * (src/r3d_band.hip:61-87). */
R3D_HD uint8_t f32_to_e4m3(float f) {
    const uint32_t u = f32_bits(f);
    const uint8_t  s = (uint8_t)((u >> 24) & 0x80u);
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(s | 0x7fu);
    if (a >= 0x43e00000u) return (uint8_t)(s | 0x7eu);
    const int e = (int)(a >> 23) - 127;
    uint32_t m = a & 0x7fffffu;
    if (e < -10) return s;
    if (e < -6) {
        const int sh = 14 - e;                               /* -6 - e + 20 */
        m |= 0x800000u;
        const uint32_t lo = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
        uint32_t q = m >> sh;
        if (lo > half || (lo == half && (q & 1u))) ++q;
        return (uint8_t)(s | q);
    }
    uint32_t q = m >> 20;
    const uint32_t lo = m & 0xfffffu;
    if (lo > 0x80000u || (lo == 0x80000u && (q & 1u))) ++q;
    int ee = e + 7;
    if (q == 8u) { q = 0; ++ee; }
    if (ee > 15 || (ee == 15 && q >= 7u)) return (uint8_t)(s | 0x7eu);
    return (uint8_t)(s | ((uint32_t)ee << 3) | q);
}

/* e2m1 -> f32: {0, .5, 1, 1.5, 2, 3, 4, 6} by the low three bits, bit 3 the sign; all
 * sixteen codes are numbers (src/r3d_mxfp4_q8x.h:17-22). Computed, not tabulated:
 * magnitude code c>=2 is (2 + (c&1)) * 2^((c>>1) - 1), c<2 is c/2. */
R3D_HD float e2m1_to_f32(uint8_t n) {
    const uint32_t c = n & 7u;
    const uint32_t s = (uint32_t)(n & 8u) << 28;
    if (c == 0u) return bits_f32(s);
    if (c == 1u) return bits_f32(s | 0x3f000000u);
    return bits_f32(s | ((126u + (c >> 1)) << 23) | ((c & 1u) << 22));
}

/* twice the e2m1 value as a small integer, the int8 arm's weight operand
 * (src/r3d_mxfp4_q8x.h:22): {0,1,2,3,4,6,8,12} and their negatives. */
R3D_HD int e2m1_x2(uint8_t n) {
    const int c = n & 7;
    const int mag = c < 2 ? c : ((2 + (c & 1)) << ((c >> 1) - 1));
    return (n & 8) ? -mag : mag;
}

/* E8M0 -> f32 (src/r3d_mxfp4_q8x.h:29-37): 2^(x-127); 0xFF is NaN; 0x00 is the f32
 * subnormal 2^-127, not zero. */
R3D_HD float e8m0_to_f32(uint8_t x) {
    if (x == 0xffu) return bits_f32(0x7fc00000u);
    if (x == 0x00u) return bits_f32(0x00400000u);
    return bits_f32((uint32_t)x << 23);
}

} /* namespace r3d */

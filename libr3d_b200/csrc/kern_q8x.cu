/* kern_q8x.cu -- the int8-per-32 activation arm of the mxfp4a8 decode band.
 *
 * Contract (src/r3d_gemm_mxfp4.hip:1143-1166, :1268-1281, :1319-1340):
 *   prologue  per (token m, 32-of-K group g): e = dec_e4m3(a); mx = max|e|;
 *             s = mx ? mx/127 : 1; x8 = (int8) rintf(e / s); SG[m,g] = s
 *   dot       p = sum x8 * (2 * e2m1)                       exact int32 over the group
 *             c = ((((float)p * SG[m,g]) * AS[m,g/4]) * 2^(x-127)) * 0.5f
 *   walk 0    per 256-of-K step T = ((c0+c1)+(c2+c3)) + ((c4+c5)+(c6+c7)); acc += T
 *   walk 1    lane (g mod 32) accumulates its groups serially; the 32 lane sums fold by a
 *             butterfly over lane xor 1, 2, 4, 8, 16
 * Both walks reproduce the reference arm's float chain bit for bit (its integer dot is
 * exact under any association).
 *
 * The reference first repacks every weight tensor into a 2.125x larger int8 plane so its
 * dot4 instruction can read bytes. Here the nibbles stay as they are in HBM: a lane owns a
 * whole 32-code group (one 16-byte load), expands the sixteen e2m1 codes to signed bytes
 * in registers with byte-permute lookups, and feeds dp4a. No plane, no cache, no extra
 * HBM traffic.
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

__global__ __launch_bounds__(256) void k_q8x_requant(
    const uint8_t* __restrict__ A, int8_t* __restrict__ X8, float* __restrict__ SG,
    const int M, const int K, const int64_t a_pitch) {
    const int cols = K >> 5;
    const int gw = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (gw >= M * cols) return;
    const int m = gw / cols, g = gw - m * cols;
    const int lane = threadIdx.x & 31;
    const float e = e4m3_to_f32(A[(int64_t)m * a_pitch + (g << 5) + lane]);
    float mx = fabsf(e);
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float s = mx ? __fdiv_rn(mx, 127.0f) : 1.0f;
    if (lane == 0) SG[(int64_t)m * cols + g] = s;
    X8[(int64_t)m * K + (g << 5) + lane] = (int8_t)rintf(__fdiv_rn(e, s));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

/* Eight e2m1 codes (one 32-bit word, code i in bits 4i..4i+3, i = k offset) -> two words of
 * signed bytes holding twice the value: lo = codes 0..3, hi = codes 4..7. Three lookups
 * per half: the positive table, the negative table, then a byte select driven by the
 * codes' sign bits. */
__device__ __forceinline__ void e2m1x8_to_s8(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t POS_LO = 0x03020100u, POS_HI = 0x0C080604u;   /* 0 1 2 3 | 4 6 8 12 */
    const uint32_t NEG_LO = 0xFDFEFF00u, NEG_HI = 0xF4F8FAFCu;   /* their negatives */
    const uint32_t mag = w & 0x77777777u;
    const uint32_t sel = ((w >> 1) & 0x44444444u) | 0x32103210u; /* byte i: 4*sign + i */
    const uint32_t p0 = prmt(POS_LO, POS_HI, mag), n0 = prmt(NEG_LO, NEG_HI, mag);
    lo = prmt(p0, n0, sel);
    const uint32_t p1 = prmt(POS_LO, POS_HI, mag >> 16), n1 = prmt(NEG_LO, NEG_HI, mag >> 16);
    hi = prmt(p1, n1, sel >> 16);
}

template <int MT, int WALK>
__global__ __launch_bounds__(128) void k_q8x_gemv(
    const R3dGemmQ p, const int8_t* __restrict__ X8, const float* __restrict__ SG) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= p.n) return;
    const int K = p.k, K32 = K >> 5;
    const int live = min(MT, p.m);
    const uint8_t* brow = (const uint8_t*)p.b + (int64_t)r * p.b_pitch;
    const uint8_t* srow = (const uint8_t*)p.b_scale + (int64_t)r * p.bs_pitch;
    const bool al16 = ((((uintptr_t)p.b) | (uintptr_t)p.b_pitch) & 15) == 0;

    float acc[MT];
    const float* as_row[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) { acc[m] = 0.0f; as_row[m] = p.a_scale + (int64_t)m * p.as_pitch; }

    /* The weight words and scale bytes of W sweeps (W * 32 groups of 32 codes) are requested back
     * to back before any of them is consumed: a lane then has W 16-byte loads in flight instead of
     * one, which is what a stream of 2.5 KB rows needs to keep HBM busy. Only the order of the loads
     * changes; every float operation keeps its place. */
    constexpr int W = 4;
    for (int gw = 0; gw < K32; gw += 32 * W) {
        uint4 wv[W];
        uint8_t sbv[W];
#pragma unroll
        for (int d = 0; d < W; ++d) {
            const int g = gw + d * 32 + lane;
            wv[d] = make_uint4(0u, 0u, 0u, 0u);
            sbv[d] = 0;
            if (g < K32) {
                if (al16) wv[d] = *(const uint4*)(brow + ((int64_t)g << 4));
                else {
                    const uint8_t* bp = brow + ((int64_t)g << 4);
                    wv[d] = make_uint4(*(const uint32_t*)bp, *(const uint32_t*)(bp + 4), *(const uint32_t*)(bp + 8),
                                       *(const uint32_t*)(bp + 12));
                }
                sbv[d] = srow[g];
            }
        }
#pragma unroll
        for (int d = 0; d < W; ++d) {
        const int g0 = gw + d * 32;
        if (g0 >= K32) break;
        const int g = g0 + lane;
        const bool on = g < K32;
        float c[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) c[m] = 0.0f;
        if (on) {
            const uint32_t w[4] = {wv[d].x, wv[d].y, wv[d].z, wv[d].w};
            uint32_t s8[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) e2m1x8_to_s8(w[i], s8[2 * i], s8[2 * i + 1]);
            const float sc = e8m0_to_f32(sbv[d]);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < live) {
                    /* offsets fit 32 bits: M <= 8 rows of at most 2^20 columns */
                    const uint4* xp = (const uint4*)(X8 + (m * K + (g << 5)));
                    const uint4 xa = __ldg(xp), xb = __ldg(xp + 1);
                    int pp = __dp4a((int)xa.x, (int)s8[0], 0);
                    pp = __dp4a((int)xa.y, (int)s8[1], pp);
                    pp = __dp4a((int)xa.z, (int)s8[2], pp);
                    pp = __dp4a((int)xa.w, (int)s8[3], pp);
                    pp = __dp4a((int)xb.x, (int)s8[4], pp);
                    pp = __dp4a((int)xb.y, (int)s8[5], pp);
                    pp = __dp4a((int)xb.z, (int)s8[6], pp);
                    pp = __dp4a((int)xb.w, (int)s8[7], pp);
                    float v = __fmul_rn((float)pp, __ldg(SG + (m * K32 + g)));
                    v = __fmul_rn(v, __ldg(as_row[m] + (g >> 2)));
                    v = __fmul_rn(v, sc);
                    c[m] = __fmul_rn(v, 0.5f);
                }
            }
        }
        if (WALK == 0) {
            /* octet = one 256-of-K step; the gate K % 256 == 0 keeps octets whole */
            const int nstep = min(4, (K32 - g0) >> 3);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float v = c[m];
                v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
                v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
                v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float t = __shfl_sync(0xffffffffu, v, 8 * j);
                    if (j < nstep) acc[m] = __fadd_rn(acc[m], t);
                }
            }
        } else {
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (on) acc[m] = __fadd_rn(acc[m], c[m]);
        }
    }
    }
    if (WALK == 1) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[m];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1)
                v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
            acc[m] = v;
        }
    }
    if (lane == 0) {
        uint16_t* Y = (uint16_t*)p.y;
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < live) Y[(int64_t)m * p.y_pitch + r] = f32_to_bf16(acc[m]);
    }
}

int q8x_requant(const R3dGemmQ& p, int8_t* x8, float* sg, cudaStream_t st) {
    const unsigned grid = (unsigned)(((int64_t)p.m * (p.k >> 5) + 7) / 8);
    count_launch();
    k_q8x_requant<<<grid, 256, 0, st>>>((const uint8_t*)p.a, x8, sg, p.m, p.k, p.a_pitch);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

int q8x_gemv(const R3dGemmQ& p, const int8_t* x8, const float* sg, int walk, cudaStream_t st) {
    if (p.m < 1 || p.m > 8 || (p.k & 255) || p.k > (1 << 20)) return RAD_E_UNSUPPORTED;   /* 32-bit offsets in the kernel */
    if ((((uintptr_t)p.b) | (uintptr_t)p.b_pitch) & 3) return RAD_E_UNSUPPORTED;
    const int mt = p.m <= 1 ? 1 : p.m <= 2 ? 2 : p.m <= 4 ? 4 : 8;
    const dim3 grid((unsigned)((p.n + 3) / 4));
    count_launch();
#define R3D_Q8X(MT_)                                                            \
    do { if (walk) k_q8x_gemv<MT_, 1><<<grid, 128, 0, st>>>(p, x8, sg);          \
         else      k_q8x_gemv<MT_, 0><<<grid, 128, 0, st>>>(p, x8, sg); } while (0)
    switch (mt) {
        case 1: R3D_Q8X(1); break;
        case 2: R3D_Q8X(2); break;
        case 4: R3D_Q8X(4); break;
        default: R3D_Q8X(8); break;
    }
#undef R3D_Q8X
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

} /* namespace r3d */

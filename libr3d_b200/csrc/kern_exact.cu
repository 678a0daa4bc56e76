/* kern_exact.cu -- the oracle-order arm of every band.
 *
 * These kernels perform the float operations of libr3d's stated arithmetic in exactly the
 * stated order, so their output is bit-identical to a scalar CPU walk of the same rule:
 *   fp8a8    src/r3d_gemm_fp8a8.hip:9-15   per 128-of-K group: ascending f32 sum of exact
 *            products, then acc += (sub * sa) * sb
 *   mxfp4a8  src/r3d_gemm_mxfp4.hip:14-15  per 32-of-K group: ascending f32 sum, then
 *            acc += (sub * sa[g/4]) * 2^(x-127)
 *   logits   src/r3d_gemm_logits.hip:5-9   w = code * scale rounded once, one fma chain
 *            per output over ascending k
 * They accept any alignment and any legal shape, which makes them the arm every other
 * kernel is cross-checked against on the device and the fallback for geometries the
 * streaming arms cannot take. Speed is secondary: a lane owns whole scale groups so the
 * group sum needs no cross-lane step, and the 32 group terms of one sweep are then added
 * in group order through shuffles (each lane performs the same additions).
 *
 * Build with -fmad=false: a contracted mul+add would be a different rounding.
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

__device__ __forceinline__ float ld_scale_any(const void* base, int64_t idx, int dt) {
    if (dt == RAD_F32) return ((const float*)base)[idx];
    if (dt == RAD_F16) return f16_to_f32(((const uint16_t*)base)[idx]);
    return bf16_to_f32(((const uint16_t*)base)[idx]);
}

/* column of a scale grid with `cols` columns that covers 128-of-K chunk c of nchunk */
__device__ __forceinline__ int scale_col(int c, int cols, int nchunk) {
    return cols == nchunk ? c : (cols == 1 ? 0 : (int)((int64_t)c * cols / nchunk));
}

/* Add the 32 lane terms of one sweep to acc in lane order; lanes >= nlive hold no term. */
__device__ __forceinline__ float ordered_add(float acc, float term, int nlive) {
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
        const float t = __shfl_sync(0xffffffffu, term, j);
        if (j < nlive) acc = __fadd_rn(acc, t);
    }
    return acc;
}

/* ------------------------------------------------------------------ fp8a8 */
template <int MT>
__global__ __launch_bounds__(128) void k_fp8a8_exact(const R3dGemmQ p, const int m0) {
    __shared__ float lut[256];
    for (int i = threadIdx.x; i < 256; i += 128) lut[i] = e4m3_to_f32((uint8_t)i);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= p.n) return;
    const int live = min(MT, p.m - m0);
    const int ngrp = p.k >> 7;
    const uint8_t* A = (const uint8_t*)p.a;
    const uint8_t* brow = (const uint8_t*)p.b + (int64_t)r * p.b_pitch;
    const int64_t srow = p.rblk > 1 ? r / p.rblk : r;

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    for (int g0 = 0; g0 < ngrp; g0 += 32) {
        const int g = g0 + lane;
        float term[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) term[m] = 0.0f;
        if (g < ngrp) {
            float part[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) part[m] = 0.0f;
            const uint8_t* bw = brow + ((int64_t)g << 7);
            for (int s = 0; s < 128; ++s) {
                const float b = lut[bw[s]];
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < live) {
                        const float a = lut[A[(int64_t)(m0 + m) * p.a_pitch + ((int64_t)g << 7) + s]];
                        part[m] = __fadd_rn(part[m], __fmul_rn(a, b));
                    }
            }
            const float sb = ld_scale_any(p.b_scale,
                                          srow * p.bs_pitch + scale_col(g, p.bs_cols, ngrp),
                                          p.bs_dtype);
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < live) {
                    const float sa = p.a_scale[(int64_t)(m0 + m) * p.as_pitch +
                                               scale_col(g, p.as_cols, ngrp)];
                    term[m] = __fmul_rn(__fmul_rn(part[m], sa), sb);
                }
        }
        const int nlive = min(32, ngrp - g0);
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = ordered_add(acc[m], term[m], nlive);
    }
    if (lane == 0) {
        uint16_t* Y = (uint16_t*)p.y;
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < live) Y[(int64_t)(m0 + m) * p.y_pitch + r] = f32_to_bf16(acc[m]);
    }
}

/* ------------------------------------------------------------------ mxfp4a8 */
/* MX8: the activation's scale is one E8M0 byte per 32 of K (a_scale holds bytes, as_pitch in bytes)
 * instead of one f32 per 128 */
template <int MT, bool MX8>
__global__ __launch_bounds__(128) void k_mxfp4a8_exact(const R3dGemmQ p, const int m0) {
    __shared__ float lut[256];
    for (int i = threadIdx.x; i < 256; i += 128) lut[i] = e4m3_to_f32((uint8_t)i);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= p.n) return;
    const int live = min(MT, p.m - m0);
    const int ngrp = (p.k + 31) >> 5;
    const int n128 = (p.k + 127) >> 7;
    const uint8_t* A = (const uint8_t*)p.a;
    const uint8_t* brow = (const uint8_t*)p.b + (int64_t)r * p.b_pitch;
    const uint8_t* srow = (const uint8_t*)p.b_scale + (int64_t)r * p.bs_pitch;

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    for (int g0 = 0; g0 < ngrp; g0 += 32) {
        const int g = g0 + lane;
        float term[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) term[m] = 0.0f;
        if (g < ngrp) {
            float part[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) part[m] = 0.0f;
            const int k0 = g << 5;
            const int kn = min(32, p.k - k0);
            for (int j = 0; j < kn; ++j) {
                const uint8_t byte = brow[(k0 + j) >> 1];
                const float w = e2m1_to_f32((j & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15));
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < live) {
                        const float a = lut[A[(int64_t)(m0 + m) * p.a_pitch + k0 + j]];
                        part[m] = __fadd_rn(part[m], __fmul_rn(a, w));
                    }
            }
            const float sc = e8m0_to_f32(srow[g]);
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < live) {
                    const float sa = MX8 ? e8m0_to_f32(((const uint8_t*)p.a_scale)[(int64_t)(m0 + m) * p.as_pitch + g])
                                         : p.a_scale[(int64_t)(m0 + m) * p.as_pitch +
                                                     scale_col(g >> 2, p.as_cols, n128)];
                    term[m] = __fmul_rn(__fmul_rn(part[m], sa), sc);
                }
        }
        const int nlive = min(32, ngrp - g0);
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = ordered_add(acc[m], term[m], nlive);
    }
    if (lane == 0) {
        uint16_t* Y = (uint16_t*)p.y;
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < live) Y[(int64_t)(m0 + m) * p.y_pitch + r] = f32_to_bf16(acc[m]);
    }
}

/* ------------------------------------------------------------------ logits
 * One thread per head row: the oracle's single fma chain cannot be split and stay
 * bit-identical. */
template <int MT>
__global__ __launch_bounds__(128) void k_logits_exact(const R3dLogits p, const int m0) {
    __shared__ float lut[256];
    for (int i = threadIdx.x; i < 256; i += 128) lut[i] = e4m3_to_f32((uint8_t)i);
    __syncthreads();
    const int n = blockIdx.x * 128 + threadIdx.x;
    if (n >= p.n) return;
    const int live = min(MT, p.m - m0);
    const uint16_t* X = (const uint16_t*)p.x;
    const uint8_t* crow = (const uint8_t*)p.codes + (int64_t)n * p.code_pitch;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    if (p.head_fmt == 0) {
        const int64_t sbase = (int64_t)(n / p.br) * p.scale_pitch;
        for (int k = 0; k < p.k; ++k) {
            const float sv = ld_scale_any(p.scale, sbase + (k >> 7), p.scale_dtype);
            const float w = __fmul_rn(lut[crow[k]], sv);
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < live)
                    acc[m] = __fmaf_rn(bf16_to_f32(X[(int64_t)(m0 + m) * p.x_pitch + k]), w, acc[m]);
        }
    } else {
        const uint8_t* srow = (const uint8_t*)p.scale + (int64_t)n * p.scale_pitch;
        for (int k = 0; k < p.k; ++k) {
            const uint8_t byte = crow[k >> 1];
            const float w = __fmul_rn(
                e2m1_to_f32((k & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15)),
                e8m0_to_f32(srow[k >> 5]));
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < live)
                    acc[m] = __fmaf_rn(bf16_to_f32(X[(int64_t)(m0 + m) * p.x_pitch + k]), w, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
        if (m < live) {
            if (p.y_dtype == RAD_F32)
                ((float*)p.y)[(int64_t)(m0 + m) * p.y_pitch + n] = acc[m];
            else
                ((uint16_t*)p.y)[(int64_t)(m0 + m) * p.y_pitch + n] = f32_to_bf16(acc[m]);
        }
}

/* ------------------------------------------------------------------ quant_act_fp8
 * src/r3d_band.hip:119-153. One block per (row, group). */
__global__ __launch_bounds__(128) void k_quant_act_fp8(
    const void* __restrict__ x, const int x_dtype, const int64_t x_pitch,
    uint8_t* __restrict__ q, const int64_t q_pitch, float* __restrict__ scale,
    const int64_t s_pitch, const int n, const int group, const int ngrp) {
    __shared__ float red[4];
    __shared__ float s_sc;
    const int row = blockIdx.x / ngrp, gi = blockIdx.x - row * ngrp;
    const int k0 = gi * group, k1 = min(k0 + group, n);
    auto ld = [&](int k) -> float {
        return x_dtype == RAD_F32 ? ((const float*)x)[(int64_t)row * x_pitch + k]
                                  : bf16_to_f32(((const uint16_t*)x)[(int64_t)row * x_pitch + k]);
    };
    float amax = 0.0f;
    for (int k = k0 + threadIdx.x; k < k1; k += 128) {
        const float m = fabsf(ld(k));
        if (m > amax) amax = m;                 /* strict >: NaN never wins */
    }
    for (int off = 16; off; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, amax, off);
        if (o > amax) amax = o;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = red[0];
        for (int w = 1; w < 4; ++w) if (red[w] > r) r = red[w];
        const float sc = r > 0.0f ? __fmul_rn(r, 1.0f / 448.0f) : 1.0f;
        s_sc = sc;
        scale[(int64_t)row * s_pitch + gi] = sc;
    }
    __syncthreads();
    const float inv = __fdiv_rn(1.0f, s_sc);
    for (int k = k0 + threadIdx.x; k < k1; k += 128) {
        float c = __fmul_rn(ld(k), inv);
        if (c > 448.0f) c = 448.0f;
        if (c < -448.0f) c = -448.0f;
        q[(int64_t)row * q_pitch + k] = f32_to_e4m3(c);
    }
}

/* ------------------------------------------------------------------ gated activation quantiser
 * The epilogue of gemm_nt_q_gated (src/r3d_gemm_fp8a8.hip:700-825 of libr3d, itself
 * src/r3d_band.hip:167-235): one block per (group, row) of the gate_up plane [M, 2n], gate half
 * first; per group of <= g columns the gated value h = bf16((silu ? gt*sg : sg) * up),
 * sg = 1/(1 + (float)exp((double)-gt)), its amax (strict >, NaN never wins), the dequant scale
 * amax/448 and the saturating RTNE e4m3 codes of h/scale. */
__global__ __launch_bounds__(128) void k_gated_quant_fp8(
    const void* __restrict__ gu, const int gu_dtype, const int64_t gu_pitch, uint8_t* __restrict__ q, const int64_t q_pitch,
    float* __restrict__ scale, const int64_t s_pitch, void* __restrict__ ob, const int ob_dtype,
    const int64_t ob_pitch, const int n, const int g, const int ngrp, const int silu) {
    /* one block per (group, row): the double-precision exp behind the sigmoid is the cost, so the
     * groups of a row run side by side and each gated value is computed once (kept in registers
     * when the group has at most 512 columns, recomputed for the code pass otherwise) */
    __shared__ float red[4];
    const int64_t row = blockIdx.y;
    const int gi = blockIdx.x;
    const uint16_t* gr = (const uint16_t*)gu + row * gu_pitch;
    const float* gf = (const float*)gu + row * gu_pitch;
    auto gated = [&](int i) -> float {
        const float gt = gu_dtype == RAD_F32 ? gf[i] : bf16_to_f32(gr[i]);
        const float up = gu_dtype == RAD_F32 ? gf[n + i] : bf16_to_f32(gr[n + i]);
        const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-gt))));
        const float a = silu ? __fmul_rn(gt, sg) : sg;
        return bf16_to_f32(f32_to_bf16(__fmul_rn(a, up)));
    };
    const int k0 = gi * g, k1 = min(k0 + g, n);
    const bool keep = k1 - k0 <= 512;
    float hv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float amax = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = k0 + j * 128 + threadIdx.x;
            if (i < k1) {
                hv[j] = gated(i);
                const float m = fabsf(hv[j]);
                if (m > amax) amax = m;                 /* strict >: NaN never wins */
            }
        }
    } else {
        for (int i = k0 + threadIdx.x; i < k1; i += 128) {
            const float m = fabsf(gated(i));
            if (m > amax) amax = m;
        }
    }
    for (int off = 16; off; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, amax, off);
        if (o > amax) amax = o;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < 4; ++w) if (red[w] > r) r = red[w];
    const float sc = r > 0.0f ? __fmul_rn(r, 1.0f / 448.0f) : 1.0f;
    if (threadIdx.x == 0) scale[row * s_pitch + gi] = sc;
    const float inv = __fdiv_rn(1.0f, sc);
    auto emit = [&](int i, float h) {
        if (ob) {
            if (ob_dtype == RAD_F32) ((float*)ob)[row * ob_pitch + i] = h;
            else ((uint16_t*)ob)[row * ob_pitch + i] = f32_to_bf16(h);
        }
        float c = __fmul_rn(h, inv);
        if (c > 448.0f) c = 448.0f;
        if (c < -448.0f) c = -448.0f;
        q[row * q_pitch + i] = f32_to_e4m3(c);
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = k0 + j * 128 + threadIdx.x;
            if (i < k1) emit(i, hv[j]);
        }
    } else {
        for (int i = k0 + threadIdx.x; i < k1; i += 128) emit(i, gated(i));
    }
}

/* ------------------------------------------------------------------ rmsnorm_quant_fp8
 * src/r3d_more.hip:248-330 of libr3d. One block of 1024 threads per row; the sum of squares is
 * taken by the first 256 of them and keeps that kernel's order (thread t adds elements t, t+256, ... ascending; a shuffle-down tree inside
 * each warp; the eight warp sums added ascending by thread 0), so rs = 1/sqrt(ss/n + eps) has the
 * same bits. With a residual the bf16-narrowed sum x + res is stored first and is what the
 * variance and the norm read. h = bf16(src * rs * (w + wadd)) goes to out_bf16 and to the group
 * quantiser (strict-max amax, scale amax/448 or 1, saturating RTNE e4m3 codes of h/scale). */
__global__ __launch_bounds__(1024) void k_rmsnorm_quant_fp8(
    const uint16_t* __restrict__ x, const int64_t x_pitch, uint16_t* __restrict__ res, const int64_t r_pitch,
    const void* __restrict__ w, const int w_dtype, uint8_t* __restrict__ q, const int64_t q_pitch,
    float* __restrict__ scale, const int64_t s_pitch, void* __restrict__ ob, const int ob_dtype,
    const int64_t ob_pitch, const int n, const int g, const int ngrp, const float eps, const float wadd) {
    __shared__ float s_part[8];
    __shared__ float s_rs;
    extern __shared__ __align__(16) uint16_t s_h[];
    const int64_t row = blockIdx.x;
    const uint16_t* xr = x + row * x_pitch;
    uint16_t* rr = res ? res + row * r_pitch : nullptr;
    /* the row (or the bf16-narrowed sum row, which is also stored back) goes to shared memory with
     * 16-byte accesses where the operands allow; the ordered sums below then read shared memory,
     * so no global load waits behind a store */
    const bool vec = (n & 7) == 0 && ((((uintptr_t)xr) | (uintptr_t)(rr ? rr : xr)) & 15u) == 0;
    if (vec) {
        for (int c = threadIdx.x; c < (n >> 3); c += 1024) {
            uint4 xv = ((const uint4*)xr)[c];
            if (rr) {
                const uint4 rv = ((const uint4*)rr)[c];
                const uint32_t xa[4] = {xv.x, xv.y, xv.z, xv.w}, ra[4] = {rv.x, rv.y, rv.z, rv.w};
                uint32_t ha[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t lo = f32_to_bf16(__fadd_rn(bf16_to_f32((uint16_t)(ra[j] & 0xffffu)), bf16_to_f32((uint16_t)(xa[j] & 0xffffu))));
                    const uint32_t hi = f32_to_bf16(__fadd_rn(bf16_to_f32((uint16_t)(ra[j] >> 16)), bf16_to_f32((uint16_t)(xa[j] >> 16))));
                    ha[j] = lo | (hi << 16);
                }
                xv = make_uint4(ha[0], ha[1], ha[2], ha[3]);
                ((uint4*)rr)[c] = xv;
            }
            ((uint4*)s_h)[c] = xv;
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 1024) {
            uint16_t h = xr[i];
            if (rr) {
                h = f32_to_bf16(__fadd_rn(bf16_to_f32(rr[i]), bf16_to_f32(h)));
                rr[i] = h;
            }
            s_h[i] = h;
        }
    }
    __syncthreads();
    /* the ordered sum is the work of the first 256 threads: the order is the reference block's */
    if (threadIdx.x < 256) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < n; i += 256) {
            const float v = bf16_to_f32(s_h[i]);
            ss = __fadd_rn(ss, __fmul_rn(v, v));
        }
        for (int off = 16; off; off >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, off));
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = s_part[0];
        for (int k = 1; k < 8; ++k) r = __fadd_rn(r, s_part[k]);
        s_rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(r, (float)n), eps)));
    }
    __syncthreads();
    const float rs = s_rs;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float src = bf16_to_f32(s_h[i]);
        const float wv = __fadd_rn(w_dtype == RAD_F32 ? ((const float*)w)[i] : bf16_to_f32(((const uint16_t*)w)[i]), wadd);
        const uint16_t h = f32_to_bf16(__fmul_rn(__fmul_rn(src, rs), wv));
        if (ob) {
            if (ob_dtype == RAD_F32) ((float*)ob)[row * ob_pitch + i] = bf16_to_f32(h);
            else ((uint16_t*)ob)[row * ob_pitch + i] = h;
        }
        s_h[i] = h;
    }
    __syncthreads();
    /* one warp per group: the group's amax is order-free, the codes are per element */
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int gi = warp; gi < ngrp; gi += 32) {
        const int k0 = gi * g, k1 = min(k0 + g, n);
        float amax = 0.0f;
        for (int i = k0 + lane; i < k1; i += 32) {
            const float m = fabsf(bf16_to_f32(s_h[i]));
            if (m > amax) amax = m;
        }
        for (int off = 16; off; off >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, amax, off);
            if (o > amax) amax = o;
        }
        const float sc = amax > 0.0f ? __fmul_rn(amax, 1.0f / 448.0f) : 1.0f;
        const float inv = __fdiv_rn(1.0f, sc);
        if (lane == 0) scale[row * s_pitch + gi] = sc;
        for (int i = k0 + lane; i < k1; i += 32) {
            float c = __fmul_rn(bf16_to_f32(s_h[i]), inv);
            if (c > 448.0f) c = 448.0f;
            if (c < -448.0f) c = -448.0f;
            q[row * q_pitch + i] = f32_to_e4m3(c);
        }
    }
}

/* ------------------------------------------------------------------ launchers */

template <typename P, typename F>
static int launch_mt(F launch, const P& p) {
    /* rows in tiles of 8 tokens; a tile of fewer rides the smallest bucket that holds it
     * (the ladder rounds UP: src/r3d_gemm_fp8a8.hip:992-997) */
    for (int m0 = 0; m0 < p.m; m0 += 8) {
        const int left = p.m - m0;
        launch(left <= 1 ? 1 : left <= 2 ? 2 : left <= 4 ? 4 : 8, m0);
    }
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

int exact_fp8a8(const R3dGemmQ& p, cudaStream_t st) {
    const dim3 grid((unsigned)((p.n + 3) / 4));
    return launch_mt(
        [&](int mt, int m0) {
            count_launch();
            switch (mt) {
                case 1: k_fp8a8_exact<1><<<grid, 128, 0, st>>>(p, m0); break;
                case 2: k_fp8a8_exact<2><<<grid, 128, 0, st>>>(p, m0); break;
                case 4: k_fp8a8_exact<4><<<grid, 128, 0, st>>>(p, m0); break;
                default: k_fp8a8_exact<8><<<grid, 128, 0, st>>>(p, m0); break;
            }
        }, p);
}

int exact_mxfp4a8(const R3dGemmQ& p, cudaStream_t st) {
    const dim3 grid((unsigned)((p.n + 3) / 4));
    return launch_mt(
        [&](int mt, int m0) {
            count_launch();
            switch (mt) {
                case 1: k_mxfp4a8_exact<1, false><<<grid, 128, 0, st>>>(p, m0); break;
                case 2: k_mxfp4a8_exact<2, false><<<grid, 128, 0, st>>>(p, m0); break;
                case 4: k_mxfp4a8_exact<4, false><<<grid, 128, 0, st>>>(p, m0); break;
                default: k_mxfp4a8_exact<8, false><<<grid, 128, 0, st>>>(p, m0); break;
            }
        }, p);
}

int exact_mxfp4mx8(const R3dGemmQ& p, cudaStream_t st) {
    const dim3 grid((unsigned)((p.n + 3) / 4));
    return launch_mt(
        [&](int mt, int m0) {
            count_launch();
            switch (mt) {
                case 1: k_mxfp4a8_exact<1, true><<<grid, 128, 0, st>>>(p, m0); break;
                case 2: k_mxfp4a8_exact<2, true><<<grid, 128, 0, st>>>(p, m0); break;
                case 4: k_mxfp4a8_exact<4, true><<<grid, 128, 0, st>>>(p, m0); break;
                default: k_mxfp4a8_exact<8, true><<<grid, 128, 0, st>>>(p, m0); break;
            }
        }, p);
}

int exact_logits(const R3dLogits& p, cudaStream_t st) {
    const dim3 grid((unsigned)((p.n + 127) / 128));
    return launch_mt(
        [&](int mt, int m0) {
            count_launch();
            switch (mt) {
                case 1: k_logits_exact<1><<<grid, 128, 0, st>>>(p, m0); break;
                case 2: k_logits_exact<2><<<grid, 128, 0, st>>>(p, m0); break;
                case 4: k_logits_exact<4><<<grid, 128, 0, st>>>(p, m0); break;
                default: k_logits_exact<8><<<grid, 128, 0, st>>>(p, m0); break;
            }
        }, p);
}

int launch_quant_act_fp8(const void* x, int x_dtype, int64_t x_pitch, void* q, int64_t q_pitch,
                         float* scale, int64_t s_pitch, int rows, int n, int group,
                         cudaStream_t st) {
    if (group <= 0 || group > n) group = n;
    const int ngrp = (n + group - 1) / group;
    count_launch();
    k_quant_act_fp8<<<(unsigned)(rows * ngrp), 128, 0, st>>>(
        x, x_dtype, x_pitch, (uint8_t*)q, q_pitch, scale, s_pitch, n, group, ngrp);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

int launch_gated_quant_fp8(const void* gu, int64_t gu_pitch, void* q, int64_t q_pitch, float* scale,
                           int64_t s_pitch, void* ob, int ob_dtype, int64_t ob_pitch, int rows, int n, int g,
                           int silu, cudaStream_t st, int gu_dtype) {
    if (g <= 0 || g > n) g = n;
    const int ngrp = (n + g - 1) / g;
    count_launch();
    k_gated_quant_fp8<<<dim3((unsigned)ngrp, (unsigned)rows), 128, 0, st>>>(gu, gu_dtype, gu_pitch, (uint8_t*)q, q_pitch, scale,
                                                      s_pitch, ob, ob_dtype, ob_pitch, n, g, ngrp, silu);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

int launch_rmsnorm_quant_fp8(const void* x, int64_t x_pitch, void* res, int64_t r_pitch, const void* w, int w_dtype,
                             void* q, int64_t q_pitch, float* scale, int64_t s_pitch, void* ob, int ob_dtype,
                             int64_t ob_pitch, int rows, int n, int g, float eps, float wadd, cudaStream_t st) {
    if (g <= 0 || g > n) g = n;
    const int ngrp = (n + g - 1) / g;
    const size_t smem = (size_t)n * 2;
    static size_t attr_set = 0;
    if (smem > 48 * 1024 && smem > attr_set) {
        if (cudaFuncSetAttribute(k_rmsnorm_quant_fp8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess) return RAD_E_DEVICE;
        attr_set = smem;
    }
    count_launch();
    k_rmsnorm_quant_fp8<<<(unsigned)rows, 1024, smem, st>>>((const uint16_t*)x, x_pitch, (uint16_t*)res, r_pitch, w,
                                                           w_dtype, (uint8_t*)q, q_pitch, scale, s_pitch, ob,
                                                           ob_dtype, ob_pitch, n, g, ngrp, eps, wadd);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

} /* namespace r3d */

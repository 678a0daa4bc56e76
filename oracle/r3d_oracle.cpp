/* r3d_oracle.cpp -- CPU restatement of libr3d's quantised-matmul arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are graded against
 * and the timed CPU baseline. Nothing the plugin ships may call, link or load it.
 *
 * Each function restates one rule of the reference, in the reference's own operation
 * order, and cites the file:line of libr3d it follows. The true arbiter behind those
 * rules (radiance `libref`: ref_gemm.h quant_dot, ref_common.h e8m0_to_f32, ref_planes.h
 * ScaledRows; module codeberg.org/StillDeadcode/radiance@v1.11.0) is a third-party
 * dependency that libr3d does not vendor; the citations below are libr3d's own scalar
 * restatements of it, which is what its unit tools grade its kernels with.
 *
 * Pinning: oracle/Makefile compiles the reference's own sources of this path from where
 * they lie (src/r3d_mxfp4_q8x.h on the CPU; the band, norm, logits, fp8a8, mxfp4 and
 * rerank .hip files for the GPU through oracle/hipstub/; the w2a8 layout hooks host-only)
 * into oracle/_ref/. tests/test_oracle_codecs.py checks this file's tables, decoders and
 * e4m3 encoder against that compiled code over all codes and rounding midpoints;
 * tests/test_gpu_ref_band.py, tests/test_gpu_band_rows.py and tests/test_gpu_rerank.py run
 * the reference's kernels beside this file's rules; tests/test_oracle_gemm.py holds the
 * known-answer cases of the reference's tools (analytic unit fixture, the probe tool's
 * srand(777) fixture, decoder spot values) and an independent numpy walk of each rule.
 * Extensions the reference has no row or test for -- the mxfp4 LM head, the OCP-MX
 * activation quantiser and the mxfp4mx8 product, fp32 per-channel / per-token scale grids
 * -- are PARITY UNPINNED: the rule is fixed by this file alone. The w2a8 rule follows the
 * reference's written transcription (src/r3d_gemm_w2a8.hip:32-51); its kernels are not run.
 *
 * Build: g++ -O3 -std=c++17 -fopenmp -ffp-contract=off (no -ffast-math): mul and add stay
 * separate roundings except where fmaf is written, as the reference builds with
 * -ffp-contract=off (CMakeLists.txt:34-37).
 */
#include <vector>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bits2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f2bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

/* bf16 <-> f32: src/r3d_gemm_fp8a8.hip:101-105, src/r3d_band.hip:53-60.
 * NaN keeps its top bits and sets the quiet bit; everything else rounds to nearest even. */
inline float bf16_to_f32(uint16_t h) { return bits2f((uint32_t)h << 16); }
inline uint16_t f32_to_bf16(float f) {
    const uint32_t u = f2bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

/* f16 -> f32 by the field walk of tools/test_logits_e4m3.cpp:38-44. */
inline float f16_to_f32(uint16_t b) {
    const int s = (b >> 15) & 1, e = (b >> 10) & 0x1F, m = b & 0x3FF;
    const float sign = s ? -1.0f : 1.0f;
    if (e == 0) return sign * std::ldexp((float)m / 1024.0f, -14);
    if (e == 31) return m ? NAN : sign * INFINITY;
    return sign * (1.0f + (float)m / 1024.0f) * std::ldexp(1.0f, e - 15);
}

/* e4m3fn decode: src/r3d_gemm_fp8a8.hip:134-150 (loop-free form). 1-4-3, bias 7, no
 * infinities, S.1111.111 the only NaN, subnormals m * 2^-9, signed zero kept. */
inline float e4m3_to_f32(uint8_t b) {
    const uint32_t s = (uint32_t)(b >> 7) << 31;
    const uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
    if (e == 0u) {
        if (m == 0u) return bits2f(s);
        const float f = (float)m / 512.0f;
        return bits2f(s | (f2bits(f) & 0x7fffffffu));
    }
    if (e == 0xfu && m == 7u) return bits2f(s | 0x7fc00000u);
    return bits2f(s | ((e - 7u + 127u) << 23) | (m << 20));
}

/* e4m3 encode, round-to-nearest-even, saturating: src/r3d_band.hip:61-87. */
inline uint8_t f32_to_e4m3(float f) {
    const uint32_t u = f2bits(f);
    const uint8_t  s = (uint8_t)((u >> 24) & 0x80u);
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(s | 0x7fu);
    if (a >= 0x43e00000u) return (uint8_t)(s | 0x7eu);      /* |v| >= 448 */
    const int e = (int)(a >> 23) - 127;
    uint32_t m = a & 0x7fffffu;
    if (e < -10) return s;
    if (e < -6) {
        const int sh = -6 - e + 20;
        m |= 0x800000u;
        const uint32_t lo = m & ((1u << sh) - 1u);
        uint32_t q = m >> sh;
        const uint32_t half = 1u << (sh - 1);
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

/* e2m1 decode: magnitudes by the low three bits, bit 3 the sign; all sixteen codes are
 * numbers. tools/probe_m4_entry.cpp:22, src/r3d_mxfp4_q8x.h:17-22. */
const float kE2M1Mag[8] = { 0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f };
inline float e2m1_to_f32(uint8_t n) { return (n & 8) ? -kE2M1Mag[n & 7] : kE2M1Mag[n & 7]; }
/* the doubled integer form the int8 arm multiplies with (src/r3d_mxfp4_q8x.h:22) */
const int8_t kE2M1x2[16] = { 0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12 };

/* E8M0 decode: src/r3d_mxfp4_q8x.h:29-37. 0xFF NaN, 0x00 the subnormal 2^-127. */
inline float e8m0_to_f32(uint8_t x) {
    uint32_t u = 0x7fc00000u;
    if (x != 0xffu) u = (x == 0x00u) ? 0x00400000u : ((uint32_t)x << 23);
    return bits2f(u);
}

/* nibble k of a packed e2m1 row: low nibble = even k (src/r3d_gemm_mxfp4.hip:265-266). */
inline uint8_t nib_at(const uint8_t* row, int64_t k) {
    const uint8_t b = row[k >> 1];
    return (k & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf);
}

/* scale-grid helper: which scale column covers 128-chunk `c` when the grid has `cols`
 * columns over `nchunk` chunks. cols == nchunk is the reference grid; cols == 1 is the
 * per-token / per-channel extension (PARITY UNPINNED). */
inline int64_t scol(int64_t c, int64_t cols, int64_t nchunk) {
    return cols == nchunk ? c : (cols == 1 ? 0 : c * cols / nchunk);
}

} /* namespace */

/* ------------------------------------------------------------------ scalar codecs */
ORC_API float    orc_e4m3_to_f32(uint8_t b) { return e4m3_to_f32(b); }
ORC_API uint8_t  orc_f32_to_e4m3(float f)   { return f32_to_e4m3(f); }
/* array form of the encoder: clamp to +-448 first, as the quantisers do */
ORC_API void     orc_f32_to_e4m3_n(const float* x, int64_t n, uint8_t* q) {
    for (int64_t i = 0; i < n; ++i) {
        float c = x[i];
        if (c > 448.0f) c = 448.0f;
        if (c < -448.0f) c = -448.0f;
        q[i] = f32_to_e4m3(c);
    }
}
ORC_API float    orc_e2m1_to_f32(uint8_t n) { return e2m1_to_f32(n); }
ORC_API int      orc_e2m1_x2(uint8_t n)     { return kE2M1x2[n & 15]; }
ORC_API float    orc_e8m0_to_f32(uint8_t x) { return e8m0_to_f32(x); }
ORC_API uint16_t orc_f32_to_bf16(float f)   { return f32_to_bf16(f); }
ORC_API float    orc_bf16_to_f32(uint16_t h){ return bf16_to_f32(h); }
ORC_API float    orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* ------------------------------------------------------------------ quant_act_fp8
 * src/r3d_band.hip:119-153. Per (row, group of <= `group` columns): amax by strict `>`
 * from 0 (NaN never wins), scale = amax > 0 ? amax * (1/448) : 1, inv = 1/scale,
 * c = clamp(x * inv, +-448), code = e4m3(c). The scale is a dequant multiplier. */
ORC_API void orc_quant_act_fp8(const float* x, int64_t M, int64_t n, int64_t group,
                               uint8_t* q, float* scale) {
    if (group <= 0 || group > n) group = n;
    const int64_t ngrp = (n + group - 1) / group;
    for (int64_t r = 0; r < M; ++r)
        for (int64_t g = 0; g < ngrp; ++g) {
            const int64_t k0 = g * group, k1 = (k0 + group < n) ? k0 + group : n;
            float amax = 0.0f;
            for (int64_t k = k0; k < k1; ++k) {
                const float m = std::fabs(x[r * n + k]);
                if (m > amax) amax = m;
            }
            const float sc = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
            scale[r * ngrp + g] = sc;
            const float inv = 1.0f / sc;
            for (int64_t k = k0; k < k1; ++k) {
                float c = x[r * n + k] * inv;
                if (c > 448.0f) c = 448.0f;
                if (c < -448.0f) c = -448.0f;
                q[r * n + k] = f32_to_e4m3(c);
            }
        }
}

/* ------------------------------------------------------------------ gated activation quantiser
 * src/r3d_gemm_fp8a8.hip:700-825 (the epilogue of gemm_nt_q_gated, itself
 * src/r3d_band.hip:167-235 verbatim). Input: the bf16 gate_up plane [M, 2n], gate half first.
 * h = bf16((silu ? gt * sg : sg) * up) with sg = 1 / (1 + (float)exp((double)-gt)); per (row,
 * group of <= g columns): amax by strict `>` from 0, scale = amax > 0 ? amax * (1/448) : 1,
 * code = e4m3(clamp(h * (1/scale), +-448)). `ob`, when given, receives h as bf16. */
ORC_API void orc_gated_quant_fp8(const uint16_t* gu, int64_t M, int64_t n, int64_t g, int silu,
                                 uint8_t* q, float* scale, uint16_t* ob) {
    if (g <= 0 || g > n) g = n;
    const int64_t ngrp = (n + g - 1) / g;
    auto gated = [&](int64_t r, int64_t i) -> float {
        const float gt = bf16_to_f32(gu[r * 2 * n + i]);
        const float up = bf16_to_f32(gu[r * 2 * n + n + i]);
        const float sg = 1.0f / (1.0f + (float)std::exp((double)(-gt)));
        const float a = silu ? gt * sg : sg;
        return bf16_to_f32(f32_to_bf16(a * up));
    };
    for (int64_t r = 0; r < M; ++r)
        for (int64_t gi = 0; gi < ngrp; ++gi) {
            const int64_t k0 = gi * g, k1 = (k0 + g < n) ? k0 + g : n;
            float amax = 0.0f;
            for (int64_t i = k0; i < k1; ++i) {
                const float m = std::fabs(gated(r, i));
                if (m > amax) amax = m;
            }
            const float sc = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
            scale[r * ngrp + gi] = sc;
            const float inv = 1.0f / sc;
            for (int64_t i = k0; i < k1; ++i) {
                const float h = gated(r, i);
                if (ob) ob[r * n + i] = f32_to_bf16(h);
                float c = h * inv;
                if (c > 448.0f) c = 448.0f;
                if (c < -448.0f) c = -448.0f;
                q[r * n + i] = f32_to_e4m3(c);
            }
        }
}

/* ------------------------------------------------------------------ rmsnorm_quant_fp8
 * src/r3d_more.hip:248-330 (kernel) of libr3d, restated as a scalar walk that keeps the KERNEL's
 * summation order, because that order decides the bits of rs: the block has 256 threads, thread t
 * adds the squares of elements t, t+256, ... ascending into its own partial; inside each warp of
 * 32 threads the partials fold by a shuffle-down tree (offsets 16, 8, 4, 2, 1: lane l adds lane
 * l+off, lane 0 ends with the warp's sum); thread 0 adds the eight warp sums ascending;
 * rs = 1 / sqrtf(ss / n + eps). With a residual, sum = bf16(res + x) is stored back first and its
 * widened value is what is squared and normed. h = bf16(src * rs * (w + wadd)) (left to right, no
 * contraction) is the norm output; the codes are the group quantiser of quant_act_fp8 over h.
 * x, res, w_bits are bf16 bit patterns; w_f32 (when given) replaces w_bits. */
ORC_API void orc_rmsnorm_quant_fp8(const uint16_t* x, uint16_t* res, const uint16_t* w_bits, const float* w_f32,
                                   int64_t M, int64_t n, int64_t g, float eps, float wadd, uint8_t* q,
                                   float* scale, uint16_t* ob) {
    if (g <= 0 || g > n) g = n;
    const int64_t ngrp = (n + g - 1) / g;
    std::vector<uint16_t> h(n);
    for (int64_t r = 0; r < M; ++r) {
        float part[256];
        for (int t = 0; t < 256; ++t) {
            float ss = 0.0f;
            for (int64_t i = t; i < n; i += 256) {
                float v = bf16_to_f32(x[r * n + i]);
                if (res) {
                    const uint16_t hb = f32_to_bf16(bf16_to_f32(res[r * n + i]) + v);
                    res[r * n + i] = hb;
                    h[i] = hb;
                    v = bf16_to_f32(hb);
                }
                ss += v * v;
            }
            part[t] = ss;
        }
        float total = 0.0f;
        for (int wp = 0; wp < 8; ++wp) {
            float lane[32];
            for (int l = 0; l < 32; ++l) lane[l] = part[wp * 32 + l];
            for (int off = 16; off; off >>= 1)
                for (int l = 0; l < 32; ++l)          /* ascending l: lane l+off still holds its old value */
                    lane[l] = lane[l] + (l + off < 32 ? lane[l + off] : lane[l]);
            total = wp == 0 ? lane[0] : total + lane[0];
        }
        const float rs = 1.0f / std::sqrt(total / (float)n + eps);
        for (int64_t i = 0; i < n; ++i) {
            const float src = res ? bf16_to_f32(h[i]) : bf16_to_f32(x[r * n + i]);
            const float wv = (w_f32 ? w_f32[i] : bf16_to_f32(w_bits[i])) + wadd;
            h[i] = f32_to_bf16(src * rs * wv);
            if (ob) ob[r * n + i] = h[i];
        }
        for (int64_t gi = 0; gi < ngrp; ++gi) {
            const int64_t k0 = gi * g, k1 = (k0 + g < n) ? k0 + g : n;
            float amax = 0.0f;
            for (int64_t i = k0; i < k1; ++i) {
                const float m = std::fabs(bf16_to_f32(h[i]));
                if (m > amax) amax = m;
            }
            const float sc = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
            const float inv = 1.0f / sc;
            scale[r * ngrp + gi] = sc;
            for (int64_t i = k0; i < k1; ++i) {
                float c = bf16_to_f32(h[i]) * inv;
                if (c > 448.0f) c = 448.0f;
                if (c < -448.0f) c = -448.0f;
                q[r * n + i] = f32_to_e4m3(c);
            }
        }
    }
}

/* ------------------------------------------------------------------ row_topk
 * src/r3d_more.hip:179-236 of libr3d: per row, R rounds of argmax under the engine's one total
 * order (value descending, ties to the lower column), each round looking only at what comes
 * strictly after the previous pick in that order. A slot the row cannot fill reports id -1 and
 * value -inf. `off` is added to every reported column. The walk below is serial (ascending column),
 * so on rows that hold a NaN it is one of the orders the reference's block reduction may take;
 * without NaNs the order of the walk cannot matter. x holds bf16 bit patterns. */
ORC_API void orc_row_topk(const uint16_t* x, int64_t M, int64_t N, int64_t R, int64_t off, int32_t* idx,
                          float* val) {
    for (int64_t m = 0; m < M; ++m) {
        float pv = INFINITY;
        int64_t pi = -1;
        for (int64_t r = 0; r < R; ++r) {
            float bv = 0.0f;
            int64_t bi = -1;
            for (int64_t i = 0; i < N; ++i) {
                const float v = bf16_to_f32(x[m * N + i]);
                if (v > pv || (v == pv && i <= pi)) continue;          /* not after the previous pick */
                if (bi < 0 || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            const bool ok = bi >= 0;
            idx[m * R + r] = ok ? (int32_t)(bi + off) : -1;
            val[m * R + r] = ok ? bv : -INFINITY;
            if (ok) { pv = bv; pi = bi; }
        }
    }
}

/* ------------------------------------------------------------------ sample_argmax
 * src/r3d_sample.hip:166-173 of libr3d (argmax_kernel over r3d_block_argmax): the column of the
 * row's largest f32 logit under the same total order as row_topk (value descending, ties to the
 * lower token id), walked here serially in ascending column. */
ORC_API void orc_sample_argmax(const float* lg, int64_t M, int64_t n_vocab, int32_t* tok) {
    for (int64_t m = 0; m < M; ++m) {
        float bv = 0.0f;
        int64_t bi = -1;
        for (int64_t i = 0; i < n_vocab; ++i) {
            const float v = lg[m * n_vocab + i];
            if (bi < 0 || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        tok[m] = (int32_t)bi;
    }
}

/* ------------------------------------------------------------------ OCP-MX activation
 * quantiser (e4m3 elements, one E8M0 scale per 32 columns). PARITY UNPINNED: the
 * reference has no such quantiser. Rule: shared exponent = floor(log2(amax)) - 8 (8 is
 * e4m3's largest exponent), stored biased by 127 and clamped to [0, 254]; elements are
 * the saturating RTNE e4m3 of x * 2^-exp. An all-zero block stores exponent byte 127. */
ORC_API void orc_quant_act_mx8(const float* x, int64_t M, int64_t n, uint8_t* q,
                               uint8_t* e8) {
    const int64_t ngrp = (n + 31) / 32;
    for (int64_t r = 0; r < M; ++r)
        for (int64_t g = 0; g < ngrp; ++g) {
            const int64_t k0 = g * 32, k1 = (k0 + 32 < n) ? k0 + 32 : n;
            float amax = 0.0f;
            for (int64_t k = k0; k < k1; ++k) {
                const float m = std::fabs(x[r * n + k]);
                if (m > amax) amax = m;
            }
            int eb = 127;
            if (amax > 0.0f && std::isfinite(amax)) {
                int ex; (void)std::frexp(amax, &ex);      /* amax = f * 2^ex, f in [.5,1) */
                eb = (ex - 1) - 8 + 127;
                if (eb < 0) eb = 0;
                if (eb > 254) eb = 254;
            }
            e8[r * ngrp + g] = (uint8_t)eb;
            const float inv = std::ldexp(1.0f, 127 - eb);
            for (int64_t k = k0; k < k1; ++k) q[r * n + k] = f32_to_e4m3(x[r * n + k] * inv);
        }
}

/* ------------------------------------------------------------------ q8x activation arm
 * src/r3d_gemm_mxfp4.hip:1150-1166 (tools/bench_dot4_seed.hip:371-379): per (m, 32
 * columns) e = dec(a); mx = max|e|; s = mx ? mx/127 : 1; x8 = (int8) rintf(e / s). */
ORC_API void orc_q8x_requant(const uint8_t* A, int64_t M, int64_t K, int64_t a_pitch,
                             int8_t* X8, float* SG) {
    const int64_t cols = K >> 5;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t g = 0; g < cols; ++g) {
            float v[32], mx = 0.0f;
            for (int j = 0; j < 32; ++j) {
                v[j] = e4m3_to_f32(A[m * a_pitch + g * 32 + j]);
                mx = std::fmax(mx, std::fabs(v[j]));
            }
            const float s = mx ? mx / 127.0f : 1.0f;
            SG[m * cols + g] = s;
            for (int j = 0; j < 32; ++j)
                X8[m * K + g * 32 + j] = (int8_t)std::rint(v[j] / s);
        }
}

/* ------------------------------------------------------------------ fp8a8 quant_dot
 * src/r3d_gemm_fp8a8.hip:9-26; scalar form tools/bench_fp8_skinny.cpp:408-419.
 * Per 128-of-K group ascending: part = sum a_k * b_k (f32, ascending k, separate mul and
 * add); acc += (part * sa[m, g]) * sb[srow, g]; y = bf16(acc).
 * bs_is_f32 / as_cols == 1 / bs_cols == 1 are the extension grids (PARITY UNPINNED).
 * Yacc (optional) receives the f32 accumulator before narrowing. */
ORC_API void orc_gemm_fp8a8(const uint8_t* A, const float* AS, const uint8_t* B,
                            const void* BS, int bs_is_f32,
                            int64_t M, int64_t N, int64_t K,
                            int64_t as_cols, int64_t bs_cols, int64_t rblk,
                            uint16_t* Y, float* Yacc) {
    const int64_t ngrp = K / 128;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const int64_t sr = rblk > 1 ? r / rblk : r;
        for (int64_t t = 0; t < M; ++t) {
            float acc = 0.0f;
            for (int64_t g = 0; g < ngrp; ++g) {
                float part = 0.0f;
                const uint8_t* a = A + t * K + g * 128;
                const uint8_t* b = B + r * K + g * 128;
                for (int s = 0; s < 128; ++s) part += lut[a[s]] * lut[b[s]];
                const int64_t bi = sr * bs_cols + scol(g, bs_cols, ngrp);
                const float sb = bs_is_f32 ? ((const float*)BS)[bi]
                                           : bf16_to_f32(((const uint16_t*)BS)[bi]);
                acc += (part * AS[t * as_cols + scol(g, as_cols, ngrp)]) * sb;
            }
            if (Y) Y[t * N + r] = f32_to_bf16(acc);
            if (Yacc) Yacc[t * N + r] = acc;
        }
    }
}

/* ------------------------------------------------------------------ mxfp4a8 quant_dot
 * src/r3d_gemm_mxfp4.hip:14-15; scalar form tools/probe_m4_entry.cpp:72-91.
 * Per 32-of-K group ascending: s = sum a_k * w_k (f32); acc += (s * sa[m, g/4]) * sc
 * with sc = E8M0(x) (0xFF NaN; the probe's ldexpf(1, x-127) equals the table for every
 * other byte, 0x00 included: 2^-127 is representable as an f32 subnormal). */
ORC_API void orc_gemm_mxfp4a8(const uint8_t* A, const float* AS, const uint8_t* B,
                              const uint8_t* BS, int64_t M, int64_t N, int64_t K,
                              int64_t as_cols, uint16_t* Y, float* Yacc) {
    const int64_t bs_cols = (K + 31) / 32, n128 = (K + 127) / 128;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* brow = B + n * (K / 2);
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t g = 0; g < bs_cols; ++g) {
                float s = 0.0f;
                const int64_t kend = (g * 32 + 32 < K) ? g * 32 + 32 : K;
                for (int64_t kk = g * 32; kk < kend; ++kk)
                    s += lut[A[m * K + kk]] * e2m1_to_f32(nib_at(brow, kk));
                const float sc = e8m0_to_f32(BS[n * bs_cols + g]);
                acc += (s * AS[m * as_cols + scol(g >> 2, as_cols, n128)]) * sc;
            }
            if (Y) Y[m * N + n] = f32_to_bf16(acc);
            if (Yacc) Yacc[m * N + n] = acc;
        }
    }
}

/* ------------------------------------------------------------------ mxfp4a8, q8x arm
 * The int8 arm's own chain, bit for bit (tools/bench_dot4_seed.hip:365-401 for walk 0,
 * src/r3d_gemm_mxfp4.hip:1341-1458 for walk 1). Inputs are the requantised activation
 * (orc_q8x_requant) and the ORIGINAL nibble + E8M0 planes.
 *   p  = sum x8 * (2 * e2m1)   exact int32 over the 32-group
 *   c  = ((((float)p * SG[m,g]) * AS[m,g/4]) * sc) * 0.5f      left to right
 *   walk 0 (dot4): per 256-of-K step T = ((c0+c1)+(c2+c3)) + ((c4+c5)+(c6+c7)); acc += T
 *   walk 1 (lane map): lane t = g mod 32 accumulates its groups serially, then the 32
 *          lane sums fold by a butterfly over lane xor 1, 2, 4, 8, 16.
 * K % 256 == 0 is the arm's gate. */
ORC_API void orc_gemm_mxfp4_q8x(const int8_t* X8, const float* SG, const float* AS,
                                const uint8_t* B, const uint8_t* BS,
                                int64_t M, int64_t N, int64_t K, int64_t as_cols,
                                int walk, uint16_t* Y, float* Yacc) {
    const int64_t K32 = K >> 5;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* brow = B + n * (K / 2);
        float* c = (float*)std::malloc((size_t)K32 * sizeof(float));
        for (int64_t m = 0; m < M; ++m) {
            for (int64_t g = 0; g < K32; ++g) {
                int32_t p = 0;
                for (int j = 0; j < 32; ++j) {
                    const int64_t k = g * 32 + j;
                    p += (int32_t)X8[m * K + k] * (int32_t)kE2M1x2[nib_at(brow, k)];
                }
                const float sc = e8m0_to_f32(BS[n * K32 + g]);
                c[g] = (float)p * SG[m * K32 + g] * AS[m * as_cols + (g >> 2)] * sc * 0.5f;
            }
            float acc = 0.0f;
            if (walk == 0) {
                for (int64_t it = 0; it < (K >> 8); ++it) {
                    const float* t = c + it * 8;
                    const float v0 = (t[0] + t[1]) + (t[2] + t[3]);
                    const float v1 = (t[4] + t[5]) + (t[6] + t[7]);
                    acc += v0 + v1;
                }
            } else {
                float lane[32];
                for (int t = 0; t < 32; ++t) lane[t] = 0.0f;
                for (int64_t g = 0; g < K32; ++g) lane[g & 31] += c[g];
                for (int off = 1; off < 32; off <<= 1) {
                    float nx[32];
                    for (int t = 0; t < 32; ++t) nx[t] = lane[t] + lane[t ^ off];
                    for (int t = 0; t < 32; ++t) lane[t] = nx[t];
                }
                acc = lane[0];
            }
            if (Y) Y[m * N + n] = f32_to_bf16(acc);
            if (Yacc) Yacc[m * N + n] = acc;
        }
        std::free(c);
    }
}

/* ------------------------------------------------------------------ logits, e4m3 head
 * src/r3d_gemm_logits.hip:5-9; oracle walk tools/test_logits_e4m3.cpp:97-110.
 * w = f32(code) * f32(scale[n/br, k/128]) rounded once; acc = fma(x, w, acc), k
 * ascending. sdt: 0 bf16, 1 f16, 2 f32. Output f32. */
ORC_API void orc_logits_e4m3(const uint16_t* X, const uint8_t* codes, const void* scale,
                             int sdt, int64_t br, int64_t M, int64_t N, int64_t K,
                             float* Y) {
    const int64_t scols = (K + 127) / 128;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                const int64_t si = (n / br) * scols + (k / 128);
                const float sv = sdt == 2 ? ((const float*)scale)[si]
                               : sdt == 1 ? f16_to_f32(((const uint16_t*)scale)[si])
                                          : bf16_to_f32(((const uint16_t*)scale)[si]);
                const float wv = lut[codes[n * K + k]] * sv;
                acc = std::fmaf(bf16_to_f32(X[m * K + k]), wv, acc);
            }
            Y[m * N + n] = acc;
        }
}

/* ------------------------------------------------------------------ logits, mxfp4 head
 * PARITY UNPINNED (the reference has no mxfp4 head row). Rule: the e4m3 head's walk with
 * w = e2m1(code) * E8M0(scale[n, k/32]) (exact: a power-of-two multiple). */
ORC_API void orc_logits_mxfp4(const uint16_t* X, const uint8_t* B, const uint8_t* BS,
                              int64_t M, int64_t N, int64_t K, float* Y) {
    const int64_t K32 = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                const float wv = e2m1_to_f32(nib_at(B + n * (K / 2), k)) *
                                 e8m0_to_f32(BS[n * K32 + (k >> 5)]);
                acc = std::fmaf(bf16_to_f32(X[m * K + k]), wv, acc);
            }
            Y[m * N + n] = acc;
        }
}

/* ------------------------------------------------------------------ f64 truth twins
 * The same dequantised operands summed in double, plus sum |a*w*scales| per output: the
 * grader's cancellation floor. Not part of the reference; used only to interpret misses. */
ORC_API void orc_truth_fp8a8(const uint8_t* A, const float* AS, const uint8_t* B,
                             const void* BS, int bs_is_f32, int64_t M, int64_t N, int64_t K,
                             int64_t as_cols, int64_t bs_cols, int64_t rblk,
                             double* Yt, double* Yabs) {
    const int64_t ngrp = K / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const int64_t sr = rblk > 1 ? r / rblk : r;
        for (int64_t t = 0; t < M; ++t) {
            double acc = 0.0, ab = 0.0;
            for (int64_t g = 0; g < ngrp; ++g) {
                const int64_t bi = sr * bs_cols + scol(g, bs_cols, ngrp);
                const double sb = bs_is_f32 ? ((const float*)BS)[bi]
                                            : bf16_to_f32(((const uint16_t*)BS)[bi]);
                const double sc = (double)AS[t * as_cols + scol(g, as_cols, ngrp)] * sb;
                for (int s = 0; s < 128; ++s) {
                    const double p = (double)e4m3_to_f32(A[t * K + g * 128 + s]) *
                                     (double)e4m3_to_f32(B[r * K + g * 128 + s]) * sc;
                    acc += p; ab += std::fabs(p);
                }
            }
            Yt[t * N + r] = acc; if (Yabs) Yabs[t * N + r] = ab;
        }
    }
}

ORC_API void orc_truth_mxfp4a8(const uint8_t* A, const float* AS, const uint8_t* B,
                               const uint8_t* BS, int64_t M, int64_t N, int64_t K,
                               int64_t as_cols, double* Yt, double* Yabs) {
    const int64_t K32 = (K + 31) / 32, n128 = (K + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            double acc = 0.0, ab = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const double sc = (double)AS[m * as_cols + scol(k >> 7, as_cols, n128)] *
                                  (double)e8m0_to_f32(BS[n * K32 + (k >> 5)]);
                const double p = (double)e4m3_to_f32(A[m * K + k]) *
                                 (double)e2m1_to_f32(nib_at(B + n * (K / 2), k)) * sc;
                acc += p; ab += std::fabs(p);
            }
            Yt[m * N + n] = acc; if (Yabs) Yabs[m * N + n] = ab;
        }
}

/* ------------------------------------------------------------------ gemm_nt_q @ w2a8 (the draft head)
 * src/r3d_gemm_w2a8.hip:32-51 of libr3d (its transcription of libref's gemm_zp, ZP_I8_ROW arm):
 *   G = K / 128; mpad = ceil(M/16)*16; q[n][k] = (B[n][k>>2] >> (2*(k&3))) & 3   (raw 0..3)
 *   A[m][k] = a[m][step_pos(k)], step_pos swaps bits 2 and 3 of k (quant_act_i8's storage order)
 *   per (m, n): acc = 0; for g ascending: is = sum_{k in g} A[m][k] * q[n][k]  (exact integer)
 *       sub = (float)is - ((float)z[n][g] * a_sum[g*mpad + m]);  acc += (sub * sa[m]) * sb[n][g]
 *   y = bf16(acc).  z is u8 (or u4, low nibble first), sb f16 widened exactly. */
static inline int w2_step_pos(int64_t k) { return (int)((k & ~12) | ((k & 4) << 1) | ((k & 8) >> 1)); }

ORC_API void orc_gemm_w2a8(const int8_t* A, const float* AS, const uint8_t* B, const uint16_t* SC_f16,
                           const uint8_t* ZP, int zp_u4, const float* ASUM, int64_t M, int64_t N, int64_t K,
                           uint16_t* Y, float* Yacc) {
    const int64_t G = K / 128, mpad = (M + 15) / 16 * 16;
    const int64_t zp_pitch = zp_u4 ? (G + 1) / 2 : G;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* crow = B + n * (K / 4);
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t g = 0; g < G; ++g) {
                int64_t is = 0;
                for (int64_t k = g * 128; k < g * 128 + 128; ++k) {
                    const int q = (crow[k >> 2] >> (2 * (k & 3))) & 3;
                    is += (int64_t)A[m * K + w2_step_pos(k)] * q;
                }
                const uint8_t zb = ZP[n * zp_pitch + (zp_u4 ? g >> 1 : g)];
                const int z = zp_u4 ? ((zb >> (4 * (g & 1))) & 15) : zb;
                const float zs = (float)z * ASUM[g * mpad + m];
                const float sub = (float)is - zs;
                const float t = sub * AS[m];
                acc += t * f16_to_f32(SC_f16[n * G + g]);
            }
            if (Y) Y[m * N + n] = f32_to_bf16(acc);
            if (Yacc) Yacc[m * N + n] = acc;
        }
    }
}

/* quant_act_i8's group sums as the band's a_sum operand: [K/128][mpad] f32, group-major, the sum of the
 * row's int8 codes over each 128 of K in COLUMN order (src/r3d_gemm_w2a8.hip:21, tools/bench_w2a8.cpp:78-84) */
ORC_API void orc_w2a8_group_sums(const int8_t* A, int64_t M, int64_t K, float* ASUM) {
    const int64_t G = K / 128, mpad = (M + 15) / 16 * 16;
    for (int64_t i = 0; i < G * mpad; ++i) ASUM[i] = 0.0f;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t g = 0; g < G; ++g) {
            float s = 0.0f;
            for (int64_t k = g * 128; k < g * 128 + 128; ++k) s += (float)A[m * K + w2_step_pos(k)];
            ASUM[g * mpad + m] = s;
        }
}

/* ------------------------------------------------------------------ logit_rerank, joined e4m3 head
 * src/r3d_logit_rerank_e4m3.hip:22-39 of libr3d (its statement of libref's ref_logit_rerank): per row
 * m and candidate r with global id g, local = g - vocab_off; g < 0 or local outside [0, n_vocab) is
 * a pad (id -1, value -inf); else acc (double) over k ascending, no FMA:
 *   hv = f32(code[local][k]) * scale[local/br][k/128]  (one f32 rounding)
 *   acc += (double) x[m][k] * (double) hv;   score = (float) acc
 * then R rounds of selection: largest value, ties to the LOWER id, pads last. x is given widened
 * to f32 (bf16 widens exactly), scale widened to f32. */
ORC_API void orc_logit_rerank_e4m3(const float* X, const uint8_t* codes, const float* scale,
                                   int64_t scale_cols, int br, const int32_t* in, int64_t M, int64_t R,
                                   int64_t K, int64_t NV, int64_t voff, int32_t* idx, float* val,
                                   float* pairs) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        int32_t sid[64]; float ssc[64]; bool used[64];
        for (int64_t r = 0; r < R; ++r) {
            const int64_t g = in[m * R + r], local = g - voff;
            used[r] = false;
            if (g < 0 || local < 0 || local >= NV) { sid[r] = -1; ssc[r] = -INFINITY; continue; }
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const float hv = e4m3_to_f32(codes[local * K + k]) * scale[(local / br) * scale_cols + (k >> 7)];
                acc += (double)X[m * K + k] * (double)hv;
            }
            sid[r] = (int32_t)g; ssc[r] = (float)acc;
        }
        for (int64_t o = 0; o < R; ++o) {
            int best = -1;
            for (int c = 0; c < R; ++c) {
                if (used[c] || sid[c] < 0) continue;
                if (best < 0 || ssc[c] > ssc[best] || (ssc[c] == ssc[best] && sid[c] < sid[best])) best = c;
            }
            const int32_t oid = best >= 0 ? sid[best] : -1;
            const float ov = best >= 0 ? ssc[best] : -INFINITY;
            if (best >= 0) used[best] = true;
            idx[m * R + o] = oid; val[m * R + o] = ov;
            if (pairs) { memcpy(&pairs[(m * R + o) * 2], &oid, 4); pairs[(m * R + o) * 2 + 1] = ov; }
        }
    }
}

/* ------------------------------------------------------------------ mxfp4 weights x mxfp8 activations
 * (dtype spelling "mxfp4mx8": e2m1 + E8M0/32 weights, e4m3 + E8M0/32 activations -- the OCP-MX pair
 * the tensor core scales by itself). PARITY UNPINNED: the reference has no such band; the rule is the
 * mxfp4a8 rule (src/r3d_gemm_mxfp4.hip:14-15 of libr3d) with the activation's f32 scale per 128
 * replaced by its E8M0 scale per 32:
 *   per 32-of-K group ascending: s = sum a_k * w_k (f32); acc += (s * 2^(xa-127)) * 2^(xw-127) */
ORC_API void orc_gemm_mxfp4mx8(const uint8_t* A, const uint8_t* AE, const uint8_t* B,
                               const uint8_t* BS, int64_t M, int64_t N, int64_t K,
                               uint16_t* Y, float* Yacc) {
    const int64_t K32 = (K + 31) / 32;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* brow = B + n * (K / 2);
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t g = 0; g < K32; ++g) {
                float s = 0.0f;
                const int64_t kend = (g * 32 + 32 < K) ? g * 32 + 32 : K;
                for (int64_t kk = g * 32; kk < kend; ++kk)
                    s += lut[A[m * K + kk]] * e2m1_to_f32(nib_at(brow, kk));
                acc += (s * e8m0_to_f32(AE[m * K32 + g])) * e8m0_to_f32(BS[n * K32 + g]);
            }
            if (Y) Y[m * N + n] = f32_to_bf16(acc);
            if (Yacc) Yacc[m * N + n] = acc;
        }
    }
}

ORC_API void orc_truth_mxfp4mx8(const uint8_t* A, const uint8_t* AE, const uint8_t* B,
                                const uint8_t* BS, int64_t M, int64_t N, int64_t K,
                                double* Yt, double* Yabs) {
    const int64_t K32 = (K + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            double acc = 0.0, ab = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const double sc = (double)e8m0_to_f32(AE[m * K32 + (k >> 5)]) * (double)e8m0_to_f32(BS[n * K32 + (k >> 5)]);
                const double p = (double)e4m3_to_f32(A[m * K + k]) *
                                 (double)e2m1_to_f32(nib_at(B + n * (K / 2), k)) * sc;
                acc += p; ab += std::fabs(p);
            }
            Yt[m * N + n] = acc; if (Yabs) Yabs[m * N + n] = ab;
        }
}

/* The host threads later calls use (0 or less: leave as is). A launcher may have exported
 * OMP_NUM_THREADS=1 for its ranks; the timed baseline asks for the cores it is meant to use. */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

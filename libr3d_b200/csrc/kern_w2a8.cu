/* kern_w2a8.cu -- gemm_nt_q at the w2a8 encoding (the draft head): int8 activations with one f32 scale
 * a row, 2-bit weight codes with an f16 scale and an integer zero point per (row, 128 of K).
 *
 * Contract (src/r3d_gemm_w2a8.hip:32-51 of libr3d, its transcription of the engine's gemm_zp), bit for
 * bit: G = K / 128; mpad = ceil(M/16)*16; q[n][k] = (b[n][k>>2] >> (2*(k&3))) & 3; A[m][k] =
 * a[m][step_pos(k)] with step_pos swapping bits 2 and 3 of k (quant_act_i8 stores columns in that order);
 *   per (m, n): acc = 0; for g ascending:
 *       is  = sum_{k in g} A[m][k] * q[n][k]                          exact integer
 *       sub = (float)is - ((float)z[n][g] * a_sum[g*mpad + m])        two f32 roundings
 *       acc += (sub * sa[m]) * sb[n][g]                               two multiplies, one add
 *   y[m][n] = bf16(acc)
 * Everything before the scales is an exact integer, so any association of the k sum gives the same
 * bits; from `sub` on the operations and their order are the oracle's.
 *
 * N = 248320 rows x K = 5120 at two bits is a 318 MB stream per call: an HBM-bound GEMV for small M.
 * The kernel is built around that stream, not around a cross-lane reduction: one THREAD owns one
 * weight row and walks it 64 bytes (two scale groups, 256 codes) at a time with four 16-byte loads,
 * so every byte is read once, every 64-byte DRAM atom is consumed whole and no value ever crosses
 * lanes; a dword's sixteen codes are split into four byte-quads by shift-and-mask and meet the
 * activation in dp4a. The activation rows are staged once per block in shared memory, de-permuted
 * from step order into the order the quads come out of a dword (k = 16 j + i + 4 b lives at byte
 * 16 j + 4 i + b), so a token's sixteen bytes for a dword are one broadcast 16-byte read. The group
 * sums, the row scales and the row's (scale, zero) pairs are exact operands of the flush above.
 * M rounds up to 1, 2, 4, 8 or 16 rows per thread (rows past M hold zeros and are never stored).
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

namespace {

constexpr int kThr = 256;

struct PW2 {
    const int8_t* a; int64_t a_pitch;
    const float* as; int64_t as_pitch;
    const uint8_t* b; int64_t b_pitch;              /* bytes */
    const uint16_t* sc; int64_t sc_pitch;           /* f16 elements */
    const uint8_t* zp; int64_t zp_pitch; int u4;    /* bytes */
    const float* asum; int mpad;
    uint16_t* y; int64_t y_pitch;
    int m, n, k;
};

__device__ __forceinline__ int step_pos(int k) { return (k & ~12) | ((k & 4) << 1) | ((k & 8) >> 1); }

template <int MT>
__device__ __forceinline__ void fold_dword(const uint32_t w, const int8_t* xrow0, const int krow, const int dw, int (&is)[MT]) {
    /* quad i = codes 16 dw + i + 4 b (b = 0..3) in bytes 0..3 */
    const uint32_t q0 = w & 0x03030303u, q1 = (w >> 2) & 0x03030303u, q2 = (w >> 4) & 0x03030303u,
                   q3 = (w >> 6) & 0x03030303u;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int4 x = *(const int4*)(xrow0 + (size_t)m * krow + dw * 16);
        is[m] = __dp4a(x.x, (int)q0, is[m]);
        is[m] = __dp4a(x.y, (int)q1, is[m]);
        is[m] = __dp4a(x.z, (int)q2, is[m]);
        is[m] = __dp4a(x.w, (int)q3, is[m]);
    }
}

template <int MT, bool VEC>
__global__ void __launch_bounds__(kThr)
k_w2a8_gemv(const PW2 P) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = P.k, G = K >> 7;
    int8_t* xs = (int8_t*)smem;                                   /* [MT][K], quad order */
    float* sum_s = (float*)(smem + (size_t)MT * K);               /* [G][MT] */
    float* sa_s = sum_s + G * MT;                                 /* [MT] */
    for (int i = threadIdx.x; i < MT * K; i += kThr) {
        const int m = i / K, k = i - m * K;
        const int dst = (k & ~15) | ((k & 3) << 2) | ((k >> 2) & 3);
        xs[(size_t)m * K + dst] = m < P.m ? P.a[(int64_t)m * P.a_pitch + step_pos(k)] : (int8_t)0;
    }
    for (int i = threadIdx.x; i < G * MT; i += kThr) {
        const int g = i / MT, m = i - g * MT;
        sum_s[i] = m < P.m ? P.asum[(int64_t)g * P.mpad + m] : 0.0f;
    }
    if (threadIdx.x < MT) sa_s[threadIdx.x] = (int)threadIdx.x < P.m ? P.as[(int64_t)threadIdx.x * P.as_pitch] : 0.0f;
    __syncthreads();

    const int n = blockIdx.x * kThr + threadIdx.x;
    if (n >= P.n) return;
    const uint8_t* brow = P.b + (int64_t)n * P.b_pitch;
    const uint16_t* srow = P.sc + (int64_t)n * P.sc_pitch;
    const uint8_t* zrow = P.zp + (int64_t)n * P.zp_pitch;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    auto flush = [&](int g, const int (&is)[MT], float sb, int z) {
        const float zf = (float)z;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float sub = __fsub_rn((float)is[m], __fmul_rn(zf, sum_s[g * MT + m]));
            acc[m] = __fadd_rn(acc[m], __fmul_rn(__fmul_rn(sub, sa_s[m]), sb));
        }
    };

    int g = 0;
    if (VEC) {
        /* eight groups at a time: their f16 scales are one 16-byte load, their u8 zeros one 8-byte load */
        for (; g + 8 <= G; g += 8) {
            const uint4 s8 = __ldg((const uint4*)(srow + g));
            const uint2 z8 = __ldg((const uint2*)(zrow + g));
            const uint32_t sw[4] = {s8.x, s8.y, s8.z, s8.w};
#pragma unroll
            for (int p = 0; p < 4; ++p) {                         /* two groups = 64 bytes of codes */
                const uint4* bp = (const uint4*)(brow + (size_t)(g + 2 * p) * 32);
                const uint4 c0 = __ldg(bp), c1 = __ldg(bp + 1), c2 = __ldg(bp + 2), c3 = __ldg(bp + 3);
                const uint32_t w[16] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w,
                                        c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int is[MT];
#pragma unroll
                    for (int m = 0; m < MT; ++m) is[m] = 0;
#pragma unroll
                    for (int d = 0; d < 8; ++d) fold_dword<MT>(w[8 * h + d], xs, K, (g + 2 * p + h) * 8 + d, is);
                    const int gi = 2 * p + h;
                    const uint32_t zb = ((gi < 4 ? z8.x : z8.y) >> (8 * (gi & 3))) & 0xffu;
                    const uint16_t sh = (uint16_t)(sw[gi >> 1] >> (16 * (gi & 1)));
                    flush(g + gi, is, f16_to_f32(sh), (int)zb);
                }
            }
        }
    }
    for (; g < G; ++g) {                                          /* any alignment, any G, u4 zeros */
        int is[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) is[m] = 0;
#pragma unroll
        for (int d = 0; d < 8; ++d) fold_dword<MT>(__ldg((const uint32_t*)(brow + (size_t)g * 32) + d), xs, K, g * 8 + d, is);
        const uint8_t zb = zrow[P.u4 ? g >> 1 : g];
        const int z = P.u4 ? (zb >> (4 * (g & 1))) & 15 : zb;
        flush(g, is, f16_to_f32(srow[g]), z);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
        if (m < P.m) P.y[(int64_t)m * P.y_pitch + n] = f32_to_bf16(acc[m]);
}

template <int MT>
int launch_mt(const PW2& P, bool vec, cudaStream_t st) {
    const size_t smem = (size_t)MT * P.k + ((size_t)(P.k >> 7) * MT + MT) * sizeof(float);
    if (smem > 200 * 1024) return RAD_E_UNSUPPORTED;
    static size_t attr_set[2][64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RAD_E_DEVICE;
    if (smem > 48 * 1024 && smem > attr_set[vec][dev]) {
        const cudaError_t e = vec ? cudaFuncSetAttribute(k_w2a8_gemv<MT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                  : cudaFuncSetAttribute(k_w2a8_gemv<MT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return RAD_E_DEVICE;
        attr_set[vec][dev] = smem;
    }
    const unsigned grid = (unsigned)((P.n + kThr - 1) / kThr);
    count_launch();
    if (vec) k_w2a8_gemv<MT, true><<<grid, kThr, smem, st>>>(P);
    else k_w2a8_gemv<MT, false><<<grid, kThr, smem, st>>>(P);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

} /* namespace */

int launch_gemm_w2a8(const R3dW2A8& q, cudaStream_t st) {
    if (q.m < 1 || q.m > 16 || q.n < 1 || q.k < 128 || (q.k & 127)) return RAD_E_UNSUPPORTED;
    PW2 P{};
    P.a = (const int8_t*)q.a; P.a_pitch = q.a_pitch;
    P.as = q.a_scale; P.as_pitch = q.as_pitch;
    P.b = (const uint8_t*)q.b; P.b_pitch = q.b_pitch;
    P.sc = (const uint16_t*)q.scale; P.sc_pitch = q.sc_pitch;
    P.zp = (const uint8_t*)q.zero; P.zp_pitch = q.zp_pitch; P.u4 = q.zero_u4;
    P.asum = q.a_sum; P.mpad = q.mpad;
    P.y = (uint16_t*)q.y; P.y_pitch = q.y_pitch;
    P.m = q.m; P.n = q.n; P.k = q.k;
    auto al = [](const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; };
    const bool vec = !q.zero_u4 && al(q.b, 16) && (q.b_pitch % 16) == 0 && al(q.scale, 16) && (q.sc_pitch % 8) == 0 &&
                     al(q.zero, 8) && (q.zp_pitch % 8) == 0;
    const int mt = q.m <= 1 ? 1 : q.m <= 2 ? 2 : q.m <= 4 ? 4 : q.m <= 8 ? 8 : 16;
    switch (mt) {
        case 1: return launch_mt<1>(P, vec, st);
        case 2: return launch_mt<2>(P, vec, st);
        case 4: return launch_mt<4>(P, vec, st);
        case 8: return launch_mt<8>(P, vec, st);
        default: return launch_mt<16>(P, vec, st);
    }
}

} /* namespace r3d */

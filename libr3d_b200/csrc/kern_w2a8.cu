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
 *
 * k_w2a8_mma (the kernel that serves aligned operands): persistent CTAs, one per SM, walk 256-row
 * tiles. A producer warp streams the tile's codes by TMA ([256 rows x 128 bytes] boxes = four scale
 * groups a stage, 128-byte swizzle, mbarrier ring); sixteen consumer warps own sixteen rows each and
 * form the exact group sums on the integer tensor-core path (mma.sync m16n8k32 s8: the sixteen rows
 * are the M axis, the tokens the N axis). A dword's sixteen codes are cut into four byte-quads by
 * shift-and-mask; quad c of a lane's two dwords is its A fragment of the group's c-th instruction,
 * and the activation rows are staged once per CTA in shared memory in exactly that order (and out of
 * quant_act_i8's step order), so a B fragment is one 8-byte read. The K order inside a group is
 * free (exact integers); the flush per group is the oracle's, two tokens per packed f32x2
 * instruction. Fragment rows are dealt to tile rows so that the swizzled 8-byte reads of a
 * half-warp fall on distinct banks. A tile's scales and zeros are staged per warp.
 *
 * k_w2a8_gemv (any alignment, any K): one THREAD owns one weight row and walks it 64 bytes (two
 * scale groups, 256 codes) at a time with four 16-byte loads; the quads meet the activation in dp4a.
 * The activation rows are staged once per block in shared memory, de-permuted from step order into
 * the order the quads come out of a dword (k = 16 j + i + 4 b lives at byte 16 j + 4 i + b), so a
 * token's sixteen bytes for a dword are one broadcast 16-byte read.
 * M rounds up to 1, 2, 4, 8 or 16 rows per thread (rows past M hold zeros and are never stored).
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"
#include <cstdlib>

namespace r3d { __device__ int g_w2_status = 0; }
#define R3D_TC_STATUS_WORD ::r3d::g_w2_status
#include "tc_common.cuh"

namespace r3d {

namespace {

using namespace tcdev;

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


/* ---------------------------------------------------------------------------------------------
 * the tensor-core kernel
 * ------------------------------------------------------------------------------------------- */
constexpr int kTileRows2 = 256;                 /* weight rows a tile */
constexpr int kCW = 16;                         /* consumer warps, sixteen rows each */
constexpr int kMmaThr = (kCW + 1) * 32;
constexpr int kStageB = kTileRows2 * 128;       /* one TMA box: 256 rows x 128 bytes (512 codes a row) */
constexpr int kMaxSt = 6;

typedef uint64_t f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
/* each half is an IEEE round-to-nearest f32 operation: the bits of the scalar instruction */
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
/* a * b rounded on its own, for a product that feeds a packed add: the assembler merges a packed
 * multiply whose only use is a packed add into one fused multiply-add (one rounding instead of the
 * contract's two; measured: a quarter of random cases differ), which it does not do to the scalar
 * forms. Written as fma(a, b, -0) the product is rounded alone (x + (-0) = x for every x, either
 * zero included) and costs the same issue slot; nz must be a (-0, -0) the assembler cannot see through. */
__device__ __forceinline__ f32x2 mul2_alone(f32x2 a, f32x2 b, f32x2 nz) {
    f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(nz)); return r;
}
__device__ __forceinline__ uint2 lds64(const void* p) { return *(const uint2*)p; }

/* D = A (16 rows x 32 k, s8) * B (32 k x 8 tokens, s8) [+ C] */
__device__ __forceinline__ void mma_s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}

struct Ring2 {
    int i = 0; uint32_t ph = 0; int n;
    __device__ explicit Ring2(int n_) : n(n_) {}
    __device__ void next() { if (++i == n) { i = 0; ph ^= 1u; } }
};

__device__ __forceinline__ uint2 lds64_at(uint32_t addr) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr)); return v;
}
__device__ __forceinline__ uint32_t lds32_at(uint32_t addr) {
    uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v;
}
/* low half of a word as f16 -> f32, high half as an unsigned integer -> f32 */
__device__ __forceinline__ float f16lo_to_f32(uint32_t w) {
    float r; asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.f32.f16 %0, lo;\n\t}" : "=f"(r) : "r"(w)); return r;
}
__device__ __forceinline__ float u16hi_to_f32(uint32_t w) {
    float r; asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f32.u16 %0, hi;\n\t}" : "=f"(r) : "r"(w)); return r;
}

/* MT = 8 or 16 token columns (one or two instructions a quad) */
template <int MT>
__global__ void __launch_bounds__(kMmaThr, 1)
k_w2a8_mma(const __grid_constant__ CUtensorMap tmW, const PW2 P, const int stages) {
    constexpr int NB = MT / 8;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int K = P.k, G = K >> 7, nst = (G + 3) >> 2;
    const int xp = K + 32;                                         /* token pitch: 8 words past a multiple of 32 banks */
    uint8_t* ring = smem;
    uint8_t* xs = ring + (size_t)stages * kStageB;                 /* [MT][xp], fragment order */
    float* sum_s = (float*)(xs + (size_t)MT * xp);                 /* [G][MT] */
    uint32_t* meta = (uint32_t*)(sum_s + G * MT);                  /* [256][G]: f16 scale | zero << 16 */
    uint64_t* full = (uint64_t*)(((uintptr_t)(meta + kTileRows2 * G) + 7) & ~(uintptr_t)7);
    uint64_t* empty = full + kMaxSt;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = (P.n + kTileRows2 - 1) / kTileRows2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kCW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kCW) {
        /* ---------------- TMA producer: the weight stream depends on nothing staged below ---------------- */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            Ring2 rg(stages);
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                for (int s = 0; s < nst; ++s) {
                    if (!mbar_wait(&empty[rg.i], rg.ph ^ 1u, 41)) { ok = false; break; }
                    mbar_expect_tx(&full[rg.i], (uint32_t)kStageB);
                    tma_load_2d(ring + (size_t)rg.i * kStageB, &tmW, s * 128, tile * kTileRows2, &full[rg.i]);
                    rg.next();
                }
            }
        }
    } else {
        /* ---------------- consumers ---------------- */
        const int ct = threadIdx.x;                                /* 0 .. 511 */
        const int k16 = K >> 4;
        for (int it = ct; it < MT * k16; it += kCW * 32) {
            /* sixteen stored bytes of one token: stored byte 4 j + c holds column 16 D + 4 swap(j) + c, where
             * swap exchanges 1 and 2; fragment word c of the sixteen = columns 16 D + 4 b + c, b = 0..3 */
            const int m = it / k16, D16 = it - m * k16;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < P.m) v = *(const uint4*)(P.a + (int64_t)m * P.a_pitch + 16 * D16);
            uint8_t* dst = xs + (size_t)m * xp + (D16 >> 3) * 128 + (D16 & 7) * 4;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t sel = (uint32_t)c | ((uint32_t)(4 + c) << 4);
                const uint32_t t01 = __byte_perm(v.x, v.z, sel);   /* columns b = 0 (stored word 0), b = 1 (stored word 2) */
                const uint32_t t23 = __byte_perm(v.y, v.w, sel);   /* columns b = 2 (stored word 1), b = 3 (stored word 3) */
                *(uint32_t*)(dst + c * 32) = __byte_perm(t01, t23, 0x5410);
            }
        }
        for (int i = ct; i < G * MT; i += kCW * 32) {
            const int g = i / MT, m = i - g * MT;
            sum_s[i] = m < P.m ? P.asum[(int64_t)g * P.mpad + m] : 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");

        const int fg = lane >> 2, t = lane & 3;                    /* fragment row group, k quarter */
        const int rho = fg < 4 ? 2 * fg : 2 * (fg - 4) + 1;        /* tile row (of the warp's sixteen) of fragment row fg */
        const int R0 = warp * 16 + rho;                            /* and R0 + 8 for fragment row fg + 8 */
        f32x2 sa2[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int t0 = nb * 8 + 2 * t;
            sa2[nb] = pk2(t0 < P.m ? P.as[(int64_t)t0 * P.as_pitch] : 0.0f,
                          t0 + 1 < P.m ? P.as[(int64_t)(t0 + 1) * P.as_pitch] : 0.0f);
        }
        /* shared-space byte addresses; everything that moves with the group is an immediate or one add */
        uint32_t a_off[4];
#pragma unroll
        for (int gg = 0; gg < 4; ++gg)
            a_off[gg] = (uint32_t)R0 * 128u + ((uint32_t)(t & 1) << 3) + ((uint32_t)((2 * gg + (t >> 1)) ^ rho) << 4);
        const uint32_t ring_a = smem_u32(ring);
        const uint32_t xb_a = smem_u32(xs) + (uint32_t)(fg * xp + t * 8);
        const uint32_t xb2_a = xb_a + 8u * (uint32_t)xp;
        const uint32_t sum_a = smem_u32(sum_s) + (uint32_t)(t * 8);
        const uint32_t m0_a = smem_u32(meta) + (uint32_t)(R0 * G * 4);
        const uint32_t m1_a = m0_a + (uint32_t)(8 * G * 4);
        uint32_t* meta_w = meta + (size_t)warp * 16 * G;

        /* both planes dense (row pitch = G) and 16-byte aligned, G <= 64: a warp's share of a tile is one
         * contiguous block of each */
        const bool dense = !P.u4 && G <= 64 && P.sc_pitch == G && P.zp_pitch == G &&
                           ((((uintptr_t)P.sc) | (uintptr_t)P.zp) & 15) == 0;
        uint4 ms[4], mz[2];
        bool have_meta = false;
        Ring2 rg(stages);
        bool alive = true;

        auto group = [&](const uint32_t sbase, const int gg, const int grp, f32x2 (&acc)[NB][2]) {
            const uint2 wa = lds64_at(sbase + a_off[gg]);
            const uint2 wb = lds64_at(sbase + a_off[gg] + 8 * 128);
            const uint32_t xg = xb_a + (uint32_t)grp * 128u, xg2 = xb2_a + (uint32_t)grp * 128u;
            int c[NB][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t a0 = (wa.x >> (2 * q)) & 0x03030303u, a1 = (wb.x >> (2 * q)) & 0x03030303u,
                               a2 = (wa.y >> (2 * q)) & 0x03030303u, a3 = (wb.y >> (2 * q)) & 0x03030303u;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const uint2 bb = lds64_at((nb ? xg2 : xg) + q * 32);
                    if (q == 0) mma_s8_first(c[nb], a0, a1, a2, a3, bb);
                    else mma_s8(c[nb], a0, a1, a2, a3, bb);
                }
            }
            const uint32_t w0 = lds32_at(m0_a + (uint32_t)grp * 4u), w1 = lds32_at(m1_a + (uint32_t)grp * 4u);
            const float sb0 = f16lo_to_f32(w0), sb1 = f16lo_to_f32(w1);
            const float z0 = u16hi_to_f32(w0), z1 = u16hi_to_f32(w1);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                /* sub = (float)is - z * a_sum (two roundings, both exact here); then (sub * sa) * sb, each
                 * product rounded on its own (scalar multiplies are never merged into the add) */
                const uint2 av = lds64_at(sum_a + (uint32_t)(grp * MT + nb * 8) * 4u);
                const float as_lo = __uint_as_float(av.x), as_hi = __uint_as_float(av.y);
                const f32x2 u0 = add2(pk2((float)c[nb][0], (float)c[nb][1]), pk2(__fmul_rn(-z0, as_lo), __fmul_rn(-z0, as_hi)));
                const f32x2 u1 = add2(pk2((float)c[nb][2], (float)c[nb][3]), pk2(__fmul_rn(-z1, as_lo), __fmul_rn(-z1, as_hi)));
                float v0l, v0h, v1l, v1h;
                upk2(mul2(u0, sa2[nb]), v0l, v0h);
                upk2(mul2(u1, sa2[nb]), v1l, v1h);
                acc[nb][0] = add2(acc[nb][0], pk2(__fmul_rn(v0l, sb0), __fmul_rn(v0h, sb0)));
                acc[nb][1] = add2(acc[nb][1], pk2(__fmul_rn(v1l, sb1), __fmul_rn(v1h, sb1)));
            }
        };

        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int64_t rowbase = (int64_t)tile * kTileRows2 + warp * 16;
            /* the warp's sixteen rows of scales and zeros, one word a (row, group): loaded a tile ahead into
             * registers when the two planes are dense (one 16-byte load a lane and 512 bytes), so that their
             * DRAM round trip hides behind the previous tile's work; any other layout (and the first tile) is
             * read here, all sixteen rows of a column in flight at once (zeros widened from u4 where packed) */
            __syncwarp();
            if (have_meta) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int e = (lane + 32 * i) * 8;               /* eight scales a 16-byte load */
                    if (e < 16 * G) {
                        const uint32_t sw[4] = {ms[i].x, ms[i].y, ms[i].z, ms[i].w};
#pragma unroll
                        for (int h = 0; h < 8; ++h)
                            ((uint16_t*)(meta_w + e + h))[0] = (uint16_t)(sw[h >> 1] >> (16 * (h & 1)));
                    }
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int e = (lane + 32 * i) * 16;              /* sixteen zeros a 16-byte load */
                    if (e < 16 * G) {
                        const uint32_t zw[4] = {mz[i].x, mz[i].y, mz[i].z, mz[i].w};
#pragma unroll
                        for (int h = 0; h < 16; ++h)
                            ((uint16_t*)(meta_w + e + h))[1] = (uint16_t)((zw[h >> 2] >> (8 * (h & 3))) & 0xffu);
                    }
                }
            } else {
                for (int g = lane; g < G; g += 32) {
                    uint16_t sv[16]; uint8_t zb[16];
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const int64_t n = rowbase + r;
                        sv[r] = 0; zb[r] = 0;
                        if (n < P.n) {
                            sv[r] = P.sc[n * P.sc_pitch + g];
                            zb[r] = P.zp[n * P.zp_pitch + (P.u4 ? g >> 1 : g)];
                        }
                    }
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const uint32_t z = P.u4 ? (uint32_t)((zb[r] >> (4 * (g & 1))) & 15) : (uint32_t)zb[r];
                        meta_w[r * G + g] = (uint32_t)sv[r] | (z << 16);
                    }
                }
            }
            have_meta = false;
            {
                const int nt = tile + (int)gridDim.x;
                const int64_t nb0 = (int64_t)nt * kTileRows2 + warp * 16;
                if (dense && nt < tiles && nb0 + 16 <= P.n) {
                    const uint4* sp = (const uint4*)(P.sc + nb0 * G);
                    const uint4* zq = (const uint4*)(P.zp + nb0 * G);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if ((lane + 32 * i) * 8 < 16 * G) ms[i] = __ldg(sp + lane + 32 * i);
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        if ((lane + 32 * i) * 16 < 16 * G) mz[i] = __ldg(zq + lane + 32 * i);
                    have_meta = true;
                }
            }
            __syncwarp();
            f32x2 acc[NB][2];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = 0ull;

            for (int s = 0; s < nst; ++s) {
                if (!mbar_wait(&full[rg.i], rg.ph, 42)) { alive = false; break; }
                const uint32_t sbase = ring_a + (uint32_t)rg.i * (uint32_t)kStageB;
                if (s * 4 + 4 <= G) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) group(sbase, gg, s * 4 + gg, acc);
                } else {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg)
                        if (s * 4 + gg < G) group(sbase, gg, s * 4 + gg, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[rg.i]);
                rg.next();
            }
            if (!alive) break;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int64_t n = rowbase + rho + 8 * h;
                    float lo, hi;
                    upk2(acc[nb][h], lo, hi);
                    const int t0 = nb * 8 + 2 * t;
                    if (n < P.n) {
                        if (t0 < P.m) P.y[(int64_t)t0 * P.y_pitch + n] = f32_to_bf16(lo);
                        if (t0 + 1 < P.m) P.y[(int64_t)(t0 + 1) * P.y_pitch + n] = f32_to_bf16(hi);
                    }
                }
        }
    }
    __syncthreads();
}

bool mma_off() {
    const char* e = getenv("R3D_W2A8_NO_MMA");
    return e && *e && *e != '0';
}

template <int MT>
int launch_mma(const PW2& P, cudaStream_t st) {
    const int G = P.k >> 7;
    const size_t fixed = (size_t)MT * (P.k + 32) + (size_t)G * MT * sizeof(float) + (size_t)kTileRows2 * G * 4 + 8 +
                         2 * kMaxSt * sizeof(uint64_t) + 1024;
    const size_t cap = 227 * 1024;
    if (fixed + 2 * (size_t)kStageB > cap) return RAD_E_UNSUPPORTED;
    int stages = (int)((cap - fixed) / kStageB);
    if (stages > kMaxSt) stages = kMaxSt;
    const size_t smem = fixed + (size_t)stages * kStageB;
    const int dev = tc_device();
    if (dev < 0) return RAD_E_DEVICE;
    static size_t attr_set[kTcMaxDevices] = {};
    if (smem > attr_set[dev]) {
        if (cudaFuncSetAttribute(k_w2a8_mma<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RAD_E_DEVICE;
        attr_set[dev] = smem;
    }
    const CUtensorMap* tw = tc_tensor_map(P.b, (uint64_t)(P.k >> 2), (uint64_t)P.n, (uint64_t)P.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)kTileRows2);
    if (!tw) return RAD_E_UNSUPPORTED;
    const int tiles = (P.n + kTileRows2 - 1) / kTileRows2;
    const int sms = tc_sm_count();
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    count_launch();
    k_w2a8_mma<MT><<<grid, kMmaThr, smem, st>>>(*tw, P, stages);
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
    /* the tensor-core kernel wants what its bulk copies and 16-byte activation reads want; q.arm =
     * R3D_ARM_EXACT or R3D_W2A8_NO_MMA=1 keep a call on the one-thread-per-row kernel */
    const bool mma = q.arm != R3D_ARM_EXACT && !mma_off() && q.k >= 512 && al(q.b, 16) && (q.b_pitch % 16) == 0 &&
                     al(q.a, 16) && (q.a_pitch % 16) == 0 && tc_have_encoder();
    if (mma) {
        const int rc = q.m <= 8 ? launch_mma<8>(P, st) : launch_mma<16>(P, st);
        if (rc != RAD_E_UNSUPPORTED) return rc;                 /* K too wide for its shared memory: walk rows below */
    }
    const int mt = q.m <= 1 ? 1 : q.m <= 2 ? 2 : q.m <= 4 ? 4 : q.m <= 8 ? 8 : 16;
    switch (mt) {
        case 1: return launch_mt<1>(P, vec, st);
        case 2: return launch_mt<2>(P, vec, st);
        case 4: return launch_mt<4>(P, vec, st);
        case 8: return launch_mt<8>(P, vec, st);
        default: return launch_mt<16>(P, vec, st);
    }
}

int tc_w2a8_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_w2_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

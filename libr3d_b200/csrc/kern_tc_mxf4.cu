/* kern_tc_mxf4.cu -- the packed-fp4 tcgen05 walk of the mxfp4a8 decode band (M <= 8).
 *
 * The unpacking tensor map of the other tcgen05 walk fetches 64-byte row segments and tops out
 * near 70 % of HBM bandwidth. This walk never unpacks: the weight plane travels as packed
 * nibbles in 128-byte row segments (a plain byte tensor map, 256 K-elements per row per stage)
 * and is consumed packed by tcgen05.mma kind::mxf4, which also applies the weights' E8M0 group
 * scales in hardware (block_scale.scale_vec::2X: one scale per 32 elements).
 *
 * kind::mxf4 wants both operands in e2m1. The e4m3 activation is therefore written as an exact
 * sum of twelve e2m1 "piece" rows per token: an e4m3 magnitude is S * 2^(e-3) with a 4-bit
 * significand S = 1b1b2b3 and -9 <= e <= 8; with j = (e+9)/3 and d = (e+9)%3
 *     hi = (1 + b1/2) * 2^e       = e2m1{1, 1.5} * 2^d * 2^(3j-9)     -> piece row j
 *     lo = (2 b2 + b3) * 2^(e-3)  = e2m1{0,.5,1,1.5,2,3,4,6} * 2^(3j-11) -> piece row 6+j
 * and every other piece of that element is zero. A small kernel (k_mxf4_split) writes the piece
 * rows once per call; they ride the MMA's N axis as separate columns and the epilogue adds them
 * with their window scales 2^(3j-9), 2^(3j-11) (exact powers of two), then applies the
 * activation's f32 scale per 128 columns -- so each product and each scale is exact and only the
 * order of the f32 additions differs from the reference walk (src/r3d_gemm_mxfp4.hip of libr3d:
 * per 32 columns (sub * sa) * 2^(x-127)).
 *
 * Scale factors in tensor memory (measured on B200): for M = 128 the MMA reads the scale bytes of
 * weight row r from TMEM lane r, column base + r/32 (base a multiple of 4), bytes
 * [a_sf_id, a_sf_id+1] of that 32-bit word for the two 32-element groups of a K=64 instruction.
 * The scale bytes come from HBM as TMA tiles of 128 rows x 32 bytes (four stages each); the
 * epilogue warps (thread = row) move each row's eight bytes per stage into tensor memory with
 * tcgen05.st. The token-side scale factors are all 2^0.
 *
 * Both kernels are launched with programmatic stream serialisation: the weight-streaming
 * kernel starts while its predecessor is still draining and requests its first ring of weight
 * and scale tiles at once -- weights are written when the model is loaded and never again, the
 * same assumption the reference's plane cache makes (src/r3d_gemm_mxfp4.hip:1879-1880) -- and
 * reads the activation side (piece rows, activation scales) only after griddepcontrol.wait.
 * R3D_NO_PDL=1 turns the early start off.
 *
 * Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 scale writers and
 * epilogue; in the split-roles form (SR, used for 3 and 4 tokens) warps 6-9 write the scale
 * factors and warps 2-5 only run the epilogue. Every wait is bounded; on expiry a status word is set and the CTA drains, frees its
 * TMEM and leaves without storing.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#define R3D_TC_STATUS_WORD ::r3d::g_tc4_status
namespace r3d { __device__ int g_tc4_status = 0; }
#include "tc_common.cuh"
#include "push.cuh"

namespace r3d {

namespace {
using namespace tcdev;

constexpr int kThreads = 192;
constexpr int kThreadsSR = 320;                    /* split roles: four more warps write the scale factors */
constexpr int kRows = 128;
constexpr int kStageK = 256;                       /* K elements per stage = 128 packed bytes per row */
constexpr int kWBytes = kRows * 128;               /* 16 KiB of weights per stage */
constexpr int kPieces = 12;
constexpr int kMaxTok = 8;

struct P4 {
    const float* as; int64_t as_pitch; int as_cols;
    const uint32_t* nanflag; int nan_blocks;       /* nanflag[t * nan_blocks + b] != 0: token t held an e4m3 NaN */
    uint16_t* y; int64_t y_pitch;
    int m, n, k;
    int ksplit, kper;                              /* CTAs per cluster = K shares per row tile; stages per share (a multiple of 4) */
    PushCfg push;                                  /* world > 0: store into every rank's gathered buffer */
};

/* window scales of the twelve piece rows */
__device__ __forceinline__ float piece_scale(int j) {
    return j < 6 ? __uint_as_float((uint32_t)(127 + 3 * j - 9) << 23)
                 : __uint_as_float((uint32_t)(127 + 3 * (j - 6) - 11) << 23);
}

/* The twelve e2m1 piece codes of one e4m3 byte, nibble p = piece row p (NaN codes give zeros:
 * the caller flags them). */
__device__ __forceinline__ uint64_t piece_codes(uint32_t b) {
    const uint32_t mag = b & 0x7fu, sgn = (b >> 4) & 8u;
    if (mag == 0x7fu || mag == 0u) return 0ull;
    uint32_t S; int e;                                   /* magnitude = S * 2^(e-3), 8 <= S <= 15 */
    if (mag >> 3) { S = 8u | (mag & 7u); e = (int)(mag >> 3) - 7; }
    else if (mag >= 4u) { S = mag << 1; e = -7; }
    else if (mag >= 2u) { S = mag << 2; e = -8; }
    else { S = 8u; e = -9; }
    const int j = (e + 9) / 3, d = (e + 9) - 3 * j;
    const uint32_t hi = sgn | ((uint32_t)(d + 1) << 1) | ((S >> 2) & 1u);
    const uint32_t kk = S & 3u;
    /* lo / 2^(3j-11) = kk * 2^(d-1) as an e2m1 code */
    const uint32_t lo_tab = d == 0 ? 0x3210u : (d == 1 ? 0x5420u : 0x7640u);
    const uint32_t lo_c = (lo_tab >> (4 * kk)) & 0xfu;
    const uint32_t lo = lo_c ? (sgn | lo_c) : 0u;
    return ((uint64_t)hi << (4 * j)) | ((uint64_t)lo << (4 * (6 + j)));
}

__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
constexpr int kScTiles = 3;                        /* ring of weight-scale tiles (4 stages each) */
constexpr int kScBytes = kRows * 32;

template <int kStages>
constexpr size_t smem_fixed() {
    return 1024 + (size_t)kScTiles * kScBytes + (4 * kStages + 8 + 2 * kScTiles) * sizeof(uint64_t) + 64;
}

/* NP: piece rows on the MMA's N axis (12 per token, padded to 16 / 32 / 48 / 96); MT: tokens
 * (1, 2, 4, 8: M rounds up, rows past M are zero-filled by the tensor map and never stored). */
/* two f32 in one 64-bit register pair and the packed fused multiply-add on them (each half an IEEE
 * fma): the twelve piece columns of a (token, group) are folded two at a time */
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r;
}

template <int NP, int MT, int kStages, bool SR>
__global__ void __launch_bounds__(SR ? kThreadsSR : kThreads)
k_tc_mxf4(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
          const __grid_constant__ CUtensorMap tmP, const P4 P) {
    constexpr int kPBytes = NP * 128;
    constexpr int kStage = kWBytes + kPBytes;
    constexpr int kBufs = NP <= 16 ? 4 : (NP <= 48 ? 2 : 1);     /* accumulator ring */
    constexpr int kAccCols = 2 * NP;                             /* two 128-column groups per stage */
    constexpr int kSfBase = kBufs * kAccCols;                    /* multiple of 4 */
    constexpr int kSfbCol = kSfBase + kStages * 8;
    constexpr int kTmemCols = 256;
    static_assert(kSfbCol + 8 <= kTmemCols && (kSfBase % 4) == 0 && kStages >= 3, "TMEM columns");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sc = smem + kStages * kStage;                        /* [kScTiles][128 rows][32 bytes] */
    uint64_t* full = (uint64_t*)(sc + kScTiles * kScBytes);       /* weights of a stage have landed */
    uint64_t* pfull = full + kStages;                             /* piece tile of a stage has landed */
    uint64_t* empty = pfull + kStages;
    uint64_t* prep = empty + kStages;                             /* scale factors of a stage are in TMEM */
    uint64_t* acc_full = prep + kStages;
    uint64_t* acc_empty = acc_full + 4;
    uint64_t* sc_full = acc_empty + 4;
    uint64_t* sc_empty = sc_full + kScTiles;
    uint32_t* tmem_slot = (uint32_t*)(sc_empty + kScTiles);
    uint32_t* nan_s = tmem_slot + 4;                              /* [8] token held an e4m3 NaN (from the split kernel's flags) */
    float* as_s = (float*)(nan_s + 8);                            /* [n128][MT] */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ks = P.ksplit;
    const int crank = ks > 1 ? (int)cluster_rank() : 0;
    const int r0 = (blockIdx.x / ks) * kRows;
    const int nk_all = P.k / kStageK;
    const int it0 = crank * P.kper;                                /* this CTA's first K stage */
    const int nk = min(P.kper, nk_all - it0);                      /* ... and how many (>= 1: the host's rule) */
    const int n128 = P.k / 128;
    const int ntile = (nk + 3) / 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1); mbar_init(&pfull[s], 1); mbar_init(&empty[s], 1); mbar_init(&prep[s], 4);
        }
        for (int b = 0; b < kBufs; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        for (int b = 0; b < kScTiles; ++b) { mbar_init(&sc_full[b], 1); mbar_init(&sc_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();                       /* barriers are initialised: the producer may start */
    dep_launch();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 1) {
        tc_fence_before();
        asm volatile("bar.sync 2, %0;" ::"n"(SR ? kThreadsSR - 32 : kThreads - 32) : "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = warp >= 1 ? *tmem_slot : 0u;
    const int q = warp & 3;                                    /* TMEM lane quarter of an epilogue warp */
    const int row = r0 + q * 32 + lane;
    float acc[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[t] = 0.0f;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer ----------------
         * Weights and their scales depend on nothing that runs before this kernel: the first ring
         * of them is requested at once. The piece tiles are the previous kernel's output and are
         * requested only after dep_wait(). */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmP) : "memory");
            auto scale_tile = [&](int tl) -> bool {
                const int r = tl % kScTiles;
                if (!mbar_wait(&sc_empty[r], ((tl / kScTiles) & 1) ^ 1, 21)) return false;
                mbar_expect_tx(&sc_full[r], (uint32_t)kScBytes);
                tma_load_2d(sc + r * kScBytes, &tmS, (it0 / 4 + tl) * 32, r0, &sc_full[r]);
                return true;
            };
            auto pieces = [&](int it) {
                const int s = it % kStages;
                mbar_expect_tx(&pfull[s], (uint32_t)kPBytes);
                tma_load_2d(smem + s * kStage + kWBytes, &tmP, (it0 + it) * 128, 0, &pfull[s]);
            };
            bool ok = scale_tile(0);
            if (ok && ntile > 1) ok = scale_tile(1);
            const int first = nk < kStages ? nk : kStages;
            for (int it = 0; it < nk && ok; ++it) {
                const int s = it % kStages;
                if (!mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1, 22)) break;
                mbar_expect_tx(&full[s], (uint32_t)kWBytes);
                tma_load_2d(smem + s * kStage, &tmW, (it0 + it) * 128, r0, &full[s]);
                if (it == first - 1) {
                    dep_wait();
                    for (int j = 0; j < first; ++j) pieces(j);
                } else if (it >= first) {
                    pieces(it);
                }
                if ((it & 3) == 3 && (it >> 2) + 2 < ntile) ok = scale_tile((it >> 2) + 2);
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (elect_one()) {
            /* instruction descriptor, block-scaled kinds: a/b format e2m1 (1), K-major operands,
             * N >> 3 at bit 17, scale format ue8m0 at bit 23, M >> 4 at bit 24, a_sf_id at bit 29 */
            const uint32_t idesc0 = (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | (1u << 23) |
                                    ((uint32_t)(kRows >> 4) << 24);
            const uint32_t idesc2 = idesc0 | (2u << 29);
            for (int it = 0; it < nk; ++it) {
                const int s = it % kStages, ab = it % kBufs;
                if (!mbar_wait(&prep[s], (it / kStages) & 1, 23)) break;
                if (!mbar_wait(&acc_empty[ab], ((it / kBufs) & 1) ^ 1, 24)) break;
                if (!mbar_wait(&full[s], (it / kStages) & 1, 25)) break;
                if (!mbar_wait(&pfull[s], (it / kStages) & 1, 29)) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(smem + s * kStage), b0 = a0 + kWBytes;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int g = i >> 1;
                    umma_mxf4(tmem_base + ab * kAccCols + g * NP, smem_desc_sw128(a0 + i * 32),
                              smem_desc_sw128(b0 + i * 32), (i & 1) ? idesc2 : idesc0,
                              tmem_base + kSfBase + s * 8 + g * 4, tmem_base + kSfbCol, (uint32_t)(i & 1));
                }
                umma_commit(&empty[s]);
                umma_commit(&acc_full[ab]);
            }
        }
    } else {
        /* ---------------- scale writers + epilogue: thread = weight row ---------------- */
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        constexpr int LEAD = kStages > 3 ? 3 : 2;
        /* the token-side scale factors are 2^0 everywhere: each warp fills its own lane quarter
         * once; the first preparation's wait::st and barrier arrival publish these stores too */
        if (!SR || warp >= 6) {
#pragma unroll
            for (int c = 0; c < 8; ++c) tmem_st1(tlane + kSfbCol + c, 0x7f7f7f7fu);
        }
        /* Preparation of stage x, LEAD stages ahead of its MMAs: this row's eight scale bytes go
         * from the scale tile in shared memory to tensor memory. */
        auto prepare = [&](int x) -> bool {
            const int s = x % kStages, r = (x >> 2) % kScTiles;
            if ((x & 3) == 0 && !mbar_wait(&sc_full[r], ((x >> 2) / kScTiles) & 1, 26)) return false;
            const uint2 sw = *(const uint2*)(sc + r * kScBytes + (q * 32 + lane) * 32 + (x & 3) * 8);
            if (!mbar_wait(&empty[s], ((x / kStages) & 1) ^ 1, 27)) return false;
            tc_fence_after();
            tmem_st1(tlane + kSfBase + s * 8 + q, sw.x);
            tmem_st1(tlane + kSfBase + s * 8 + 4 + q, sw.y);
            if ((x & 3) == 3 || x == nk - 1) { __syncwarp(); if (lane == 0) mbar_arrive(&sc_empty[r]); }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&prep[s]);
            return true;
        };
        if (SR && warp >= 6) {
            /* split roles: these four warps only write scale factors, as far ahead as the stage
             * ring allows; the epilogue warps never wait for a tensor-memory store */
            for (int x = 0; x < nk && alive; ++x) alive = prepare(x);
        } else {
        if (!SR) {
#pragma unroll
            for (int x = 0; x < LEAD; ++x)
                if (x < nk && alive) alive = prepare(x);
        }
        /* the activation scales and the NaN flags are the previous kernels' output */
        dep_wait();
        if (threadIdx.x - 64 < MT) {
            const int t = threadIdx.x - 64;
            uint32_t nan = 0u;
            if (t < P.m)
                for (int b = 0; b < P.nan_blocks; ++b) nan |= __ldg(P.nanflag + t * P.nan_blocks + b);
            nan_s[t] = nan;
        }
        /* two loads a thread in flight (one a turn of the loop measured 2.4 % slower over the M = 1, 2, 4 step:
         * this staging is on the path from the split kernel's end to the first flush) */
        for (int base = threadIdx.x - 64; base < n128 * MT; base += 2 * 128) {
            float v[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = base + u * 128;
                const int g = i / MT, t = i - g * MT;
                const int c = P.as_cols == n128 ? g : (P.as_cols == 1 ? 0 : (int)((int64_t)g * P.as_cols / n128));
                v[u] = (i < n128 * MT && t < P.m) ? __ldg(P.as + (int64_t)t * P.as_pitch + c) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (base + u * 128 < n128 * MT) as_s[base + u * 128] = v[u];
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        f32x2 wj2[kPieces / 2];
#pragma unroll
        for (int j = 0; j < kPieces / 2; ++j) wj2[j] = pk2(piece_scale(2 * j), piece_scale(2 * j + 1));
        /* the window-weighted sum of a (token, group)'s twelve piece columns, two columns an instruction */
        auto fold = [&](const float* c) -> float {
            if (MT <= 2) {
                /* one and two tokens: the scalar chain (measured: the packed form costs M = 2 a microsecond) */
                float v = c[0] * piece_scale(0);
#pragma unroll
                for (int j = 1; j < kPieces; ++j) v = fmaf(c[j], piece_scale(j), v);
                return v;
            }
            f32x2 v = mul2(pk2(c[0], c[1]), wj2[0]);
#pragma unroll
            for (int j = 1; j < kPieces / 2; ++j) v = fma2(pk2(c[2 * j], c[2 * j + 1]), wj2[j], v);
            float lo, hi;
            upk2(v, lo, hi);
            return lo + hi;
        };
        for (int it = 0; it < nk && alive; ++it) {
            if (!SR && it + LEAD < nk) { alive = prepare(it + LEAD); if (!alive) break; }
            const int ab = it % kBufs;
            if (!mbar_wait(&acc_full[ab], (it / kBufs) & 1, 28)) { alive = false; break; }
            tc_fence_after();
            constexpr int NC = (MT * kPieces + 15) / 16 * 16;       /* piece columns read per group */
            const float* sa = as_s + (2 * (it0 + it)) * MT;
            if (MT <= 2 || (MT <= 4 && !SR)) {
                /* both 128-column groups in one round trip to tensor memory */
                float c[2][NC];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const uint32_t ta = tlane + ab * kAccCols + g * NP;
                    tmem_ld16(ta, c[g]);
                    if (NC > 16) tmem_ld16(ta + 16, c[g] + 16);
                    if (NC > 32) tmem_ld16(ta + 32, c[g] + 32);
                }
                tmem_ld_wait();
                tmem_pin<NC>(c[0]);
                tmem_pin<NC>(c[1]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
#pragma unroll
                for (int t = 0; t < MT; ++t) {
#pragma unroll
                    for (int g = 0; g < 2; ++g) acc[t] += fold(c[g] + t * kPieces) * sa[g * MT + t];
                }
            } else {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    float c[NC];
                    const uint32_t ta = tlane + ab * kAccCols + g * NP;
#pragma unroll
                    for (int h = 0; h < NC / 16; ++h) tmem_ld16(ta + h * 16, c + h * 16);
                    tmem_ld_wait();
                    tmem_pin<NC>(c);
                    if (g == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[ab]);
                    }
#pragma unroll
                    for (int t = 0; t < MT; ++t) acc[t] += fold(c + t * kPieces) * sa[g * MT + t];
                }
            }
        }
        if (ks > 1 && crank != 0) {
            /* every stage of this CTA has been consumed: the stage ring is free to carry the partial
             * sums to the cluster's leader */
            float* red = (float*)smem;
#pragma unroll
            for (int t = 0; t < MT; ++t) red[t * kRows + q * 32 + lane] = alive ? acc[t] : __int_as_float(0x7fc00000);
        }
        } /* epilogue warps */
    }
    if (ks > 1) {
        cluster_sync_all();                                   /* partial sums are in place */
        if (warp >= 2 && warp < 6 && crank == 0) {
            const float* red = (const float*)smem;
            for (int r = 1; r < ks; ++r)
#pragma unroll
                for (int t = 0; t < MT; ++t) acc[t] += ld_peer_f32(red + t * kRows + q * 32 + lane, (uint32_t)r);
        }
    }
    if (warp >= 2 && warp < 6 && crank == 0 && alive && row < P.n) {
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            if (t >= P.m) break;
            const float v = nan_s[t] ? __int_as_float(0x7fc00000) : acc[t];
            if (P.push.world) push_store<uint16_t>(P.push, t, row, f32_to_bf16(v));
            else P.y[(int64_t)t * P.y_pitch + row] = f32_to_bf16(v);
        }
    }
    if (ks > 1) cluster_sync_all();                           /* peers' smem was read: they may leave */
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

/* ------------------------------------------------------------------ activation split */
constexpr int kMaxK = 32768;
__device__ __align__(256) uint8_t g_p4_pieces[kMaxTok * kPieces * (kMaxK / 2)];
__device__ uint32_t g_p4_nan[kMaxTok * (kMaxK / 256)];       /* one flag per split block (128 threads x >= 2 elements) */

/* one thread per EPT (2, 4 or 8) consecutive K elements of one token (blockIdx.y): EPT e4m3 bytes in,
 * EPT packed e2m1 nibbles out to each of the token's twelve piece rows; every block also writes its
 * "saw a NaN code" flag, set or clear, so no flag outlives the call that wrote it. The kernel sits on
 * the critical path of every call (the weight-streaming kernel waits for it), so the work per thread
 * is kept short: fewer elements per thread, more threads. */
template <int EPT>
__global__ void __launch_bounds__(128)
k_mxf4_split(const uint8_t* __restrict__ a, int64_t a_pitch, int k,
             uint8_t* __restrict__ pieces, uint32_t* __restrict__ nanflag) {
    dep_launch();
    dep_wait();                    /* the activation is the previous kernel's output, and the
                                      previous reader of the piece rows must have finished */
    const int per = k / EPT;
    const int c = blockIdx.x * 128 + threadIdx.x, t = blockIdx.y;
    bool nan = false;
    if (c < per) {
        const uint8_t* src = a + (int64_t)t * a_pitch + c * EPT;
        uint32_t raw[2] = {0u, 0u};
        if (EPT == 8) { const uint2 r = __ldg((const uint2*)src); raw[0] = r.x; raw[1] = r.y; }
        else if (EPT == 4) raw[0] = __ldg((const uint32_t*)src);
        else raw[0] = __ldg((const uint16_t*)src);
        uint32_t out[kPieces];
#pragma unroll
        for (int p = 0; p < kPieces; ++p) out[p] = 0u;
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const uint32_t b = (raw[e >> 2] >> (8 * (e & 3))) & 0xffu;
            if ((b & 0x7fu) == 0x7fu) nan = true;
            const uint64_t L = piece_codes(b);
#pragma unroll
            for (int p = 0; p < kPieces; ++p) out[p] |= (uint32_t)((L >> (4 * p)) & 0xfull) << (4 * e);
        }
        const int64_t rowb = k / 2;
#pragma unroll
        for (int p = 0; p < kPieces; ++p) {
            uint8_t* dst = pieces + (int64_t)(t * kPieces + p) * rowb + c * (EPT / 2);
            if (EPT == 8) *(uint32_t*)dst = out[p];
            else if (EPT == 4) *(uint16_t*)dst = (uint16_t)out[p];
            else *dst = (uint8_t)out[p];
        }
    }
    const int any = __syncthreads_or(nan ? 1 : 0);
    if (threadIdx.x == 0) nanflag[t * gridDim.x + blockIdx.x] = any ? 1u : 0u;
}

struct Scratch { uint8_t* pieces; uint32_t* nan; };
bool scratch(Scratch* out) {
    static Scratch per_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!per_dev[dev].pieces) {
        void *p = nullptr, *q = nullptr;
        if (cudaGetSymbolAddress(&p, g_p4_pieces) != cudaSuccess ||
            cudaGetSymbolAddress(&q, g_p4_nan) != cudaSuccess) { (void)cudaGetLastError(); return false; }
        per_dev[dev].pieces = (uint8_t*)p; per_dev[dev].nan = (uint32_t*)q;
    }
    *out = per_dev[dev];
    return true;
}

/* launch with the programmatic-serialisation attribute: the kernel may begin before its
 * predecessor in the stream has finished, and orders itself with dep_wait() */
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = tc_pdl_on() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int NP, int MT, int kStages, bool SR>
int launch_s(const CUtensorMap* tw, const CUtensorMap* ts, const CUtensorMap* tp, const P4& P, cudaStream_t st) {
    const size_t smem = smem_fixed<kStages>() + (size_t)kStages * (kWBytes + NP * 128) +
                        (size_t)(P.k / 128) * MT * sizeof(float);
    static size_t attr_set_dev[kTcMaxDevices] = {};
    const int adev = tc_device();
    if (adev < 0) return RAD_E_DEVICE;
    size_t& attr_set = attr_set_dev[adev];
    if (smem > attr_set) {
        if (cudaFuncSetAttribute(k_tc_mxf4<NP, MT, kStages, SR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return RAD_E_DEVICE;
        (void)cudaFuncSetAttribute(k_tc_mxf4<NP, MT, kStages, SR>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   (int)cudaSharedmemCarveoutMaxShared);
        attr_set = smem;
    }
    /* K shares per row tile (CTAs of one cluster), the rule measured for the other tcgen05 walk:
     * a grid near 190-250 CTAs, at most five shares; shares are whole scale tiles (4 stages) */
    P4 Q = P;
    const int tiles = (P.n + kRows - 1) / kRows, nk_all = P.k / kStageK;
    static const int forced = [] { const char* e = getenv("R3D_TC_KSPLIT"); return e ? atoi(e) : 0; }();
    int ks = forced > 0 ? forced : (5 * tc_sm_count() / 3) / (tiles > 0 ? tiles : 1);
    if (forced <= 0 && ks > 5) ks = 5;
    if (ks > 8) ks = 8;
    int per = nk_all;
    for (; ks > 1; --ks) {
        per = ((nk_all + ks - 1) / ks + 3) / 4 * 4;
        if ((ks - 1) * per < nk_all) break;                   /* every share holds at least one stage */
    }
    if (ks <= 1) { ks = 1; per = nk_all; }
    Q.ksplit = ks; Q.kper = per;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(tiles * ks)); cfg.blockDim = dim3(SR ? kThreadsSR : kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)ks; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = tc_pdl_on() ? 2 : 1;
    count_launch();
    const cudaError_t e = cudaLaunchKernelEx(&cfg, k_tc_mxf4<NP, MT, kStages, SR>, *tw, *ts, *tp, Q);
    return e == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

template <int NP, int MT, bool SR>
int launch_r(const CUtensorMap* tw, const CUtensorMap* ts, const CUtensorMap* tp, const P4& P, cudaStream_t st) {
    /* the deepest ring that still lets two CTAs share an SM */
    const size_t extra = (size_t)(P.k / 128) * MT * sizeof(float);
    const size_t stage = kWBytes + NP * 128;
    const size_t half = 233472 / 2 - 1024;
    if (smem_fixed<6>() + extra + 6 * stage <= half) return launch_s<NP, MT, 6, SR>(tw, ts, tp, P, st);
    if (smem_fixed<5>() + extra + 5 * stage <= half) return launch_s<NP, MT, 5, SR>(tw, ts, tp, P, st);
    if (smem_fixed<4>() + extra + 4 * stage <= half) return launch_s<NP, MT, 4, SR>(tw, ts, tp, P, st);
    return launch_s<NP, MT, 3, SR>(tw, ts, tp, P, st);
}

template <int NP, int MT>
int launch(const CUtensorMap* tw, const CUtensorMap* ts, const CUtensorMap* tp, const P4& P, cudaStream_t st) {
    /* split roles pay where the epilogue is long (3 or 4 tokens: measured 18.2 -> 16.5 us on
     * 27648 x 5120); with 1 or 2 tokens they change nothing. R3D_TC_SR=0|1 forces either form. */
    static const int sr = [] { const char* e = getenv("R3D_TC_SR"); return e ? atoi(e) : -1; }();
    const bool on = sr >= 0 ? sr != 0 : MT == 4;
    return on ? launch_r<NP, MT, true>(tw, ts, tp, P, st) : launch_r<NP, MT, false>(tw, ts, tp, P, st);
}

bool al(const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; }

} /* anonymous namespace */

bool tc_mxf4_ok(const R3dGemmQ& p) {
    return p.m >= 1 && p.m <= kMaxTok && p.k >= 256 && (p.k % 256) == 0 && p.k <= kMaxK &&
           al(p.b, 16) && (p.b_pitch % 16) == 0 && al(p.b_scale, 16) && (p.bs_pitch % 16) == 0 &&
           al(p.a, 8) && (p.a_pitch % 8) == 0 && p.bs_cols == p.k / 32 && tc_have_encoder();
}

/* Two launches: the activation split into e2m1 piece rows (file-scope device scratch: calls must
 * be ordered on one stream), then the weight-streaming kernel. */
int tc_mxf4(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push) {
    Scratch sc;
    if (!scratch(&sc)) return RAD_E_DEVICE;
    static const int ept = [] { const char* e = getenv("R3D_SPLIT_EPT"); const int v = e ? atoi(e) : 2;
                                return v == 8 || v == 4 ? v : 2; }();
    const int nb = (p.k / ept + 127) / 128;
    count_launch();
    const dim3 sgrid((unsigned)nb, (unsigned)p.m);
    cudaError_t se;
    if (ept == 8) se = launch_pdl(k_mxf4_split<8>, sgrid, dim3(128), 0, st, (const uint8_t*)p.a, (int64_t)p.a_pitch, (int)p.k, sc.pieces, sc.nan);
    else if (ept == 4) se = launch_pdl(k_mxf4_split<4>, sgrid, dim3(128), 0, st, (const uint8_t*)p.a, (int64_t)p.a_pitch, (int)p.k, sc.pieces, sc.nan);
    else se = launch_pdl(k_mxf4_split<2>, sgrid, dim3(128), 0, st, (const uint8_t*)p.a, (int64_t)p.a_pitch, (int)p.k, sc.pieces, sc.nan);
    if (se != cudaSuccess) return RAD_E_DEVICE;
    const int np = p.m == 1 ? 16 : (p.m == 2 ? 32 : (p.m <= 4 ? 48 : 96));
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)(p.k / 2), (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows);
    const CUtensorMap* ts = tc_tensor_map(p.b_scale, (uint64_t)(p.k / 32), (uint64_t)p.n, (uint64_t)p.bs_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows, 32u);
    const CUtensorMap* tp = tc_tensor_map(sc.pieces, (uint64_t)(p.k / 2), (uint64_t)(p.m * kPieces),
                                          (uint64_t)(p.k / 2), CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)np);
    if (!tw || !ts || !tp) return RAD_E_UNSUPPORTED;
    P4 P{};
    P.as = p.a_scale; P.as_pitch = p.as_pitch; P.as_cols = p.as_cols;
    P.nanflag = sc.nan; P.nan_blocks = nb;
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k;
    if (push) P.push = *push;
    if (p.m == 1) return launch<16, 1>(tw, ts, tp, P, st);
    if (p.m == 2) return launch<32, 2>(tw, ts, tp, P, st);
    if (p.m <= 4) return launch<48, 4>(tw, ts, tp, P, st);
    return launch<96, 8>(tw, ts, tp, P, st);
}

int tc_mxf4_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc4_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

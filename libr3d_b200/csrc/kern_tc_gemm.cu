/* kern_tc_gemm.cu -- the prefill band (M > 64) of gemm_nt_q on tcgen05: one CTA per
 * [128 weight rows x 192 tokens] output tile, looping over K in stages of 128.
 *
 * Orientation is the decode kernels': weight rows on the MMA's M axis (one TMEM lane per weight
 * row), tokens on its N axis (192 columns: two accumulator buffers plus the scale-factor columns fit
 * tensor memory, and the running sums of an epilogue thread, 64 with twelve epilogue warps, fit the register file). Both operand tiles arrive by TMA in the
 * 128-byte-swizzled layout; four K=32 MMAs per stage accumulate one 128-column group of K in
 * one TMEM buffer while the twelve epilogue warps drain the other:
 *   fp8a8    kind::f8f6f4;   acc[t] += sub128[t] * (sa[t,g] * sb[row/128,g])  (block grid), or
 *                            acc[t] += (sub128[t] * sa[t,g]) * sb[row,g]      (per-row grid)
 *   mxfp4a8  kind::mxf8f6f4.block_scale: the e2m1 nibbles are unpacked by the tensor map, the
 *            weights' E8M0 group scales (one per 32 K) are applied by the tensor core from
 *            tensor memory, and the epilogue only applies the activation's f32 scale:
 *                            acc[t] += sub128_scaled[t] * sa[t,g]
 * The reference's tile kernels make the same trade (one flush per 128 K with the scale product,
 * src/r3d_gemm_fp8a8.hip:194-335, src/r3d_gemm_mxfp4.hip:176-355 of libr3d): a tolerance-class
 * walk, graded against the oracle at 2 bf16 ulp.
 *
 * Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-13 epilogue (warp
 * w: TMEM lane quarter w & 3, token third (w - 2) / 4), warp 14 scale warp. Every wait is bounded; on expiry a status
 * word is set and the CTA drains, frees its TMEM and leaves without storing.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#define R3D_TC_STATUS_WORD ::r3d::g_tcg_status
namespace r3d { __device__ int g_tcg_status = 0; }
#include "tc_common.cuh"

namespace r3d {

namespace {
using namespace tcdev;

constexpr int kEpiParts = 3;                       /* epilogue warps per TMEM lane quarter: each takes kTok / 3 tokens */
constexpr int kEpiWarps = 4 * kEpiParts;
constexpr int kThreads = 32 * (2 + kEpiWarps + 1); /* producer, MMA, 12 epilogue warps, scale warp */
constexpr int kFs = 4;                             /* ring of per-token factor vectors */
constexpr int kRows = 128;                         /* weight rows per tile */
constexpr int kTok = 192;                          /* tokens per tile */
constexpr int kHalf = kTok / kEpiParts;            /* tokens per epilogue warp: 64 */
constexpr int kStageK = 128;
constexpr int kWBytes = kRows * kStageK;           /* 16 KiB (as laid out in shared memory) */
constexpr int kABytes = kTok * kStageK;            /* 30 KiB */
constexpr int kStage = kWBytes + kABytes;
constexpr int kStages = 5;
constexpr int kScTiles = 2;                        /* mxfp4: ring of weight-scale tiles (8 stages each) */
constexpr int kScBytes = kRows * 32;
constexpr int kSfSlots = 4;                        /* mxfp4: ring of scale-factor columns in TMEM */
constexpr int kSfBase = 2 * kTok;                  /* 384 */
constexpr int kSfbCol = kSfBase + kSfSlots * 4;    /* 400 */
constexpr int kTmemCols = 512;

enum { G_FP8 = 0, G_MXFP4 = 1, G_FP8_ROW = 2 };   /* fp8a8 block grid, mxfp4a8, fp8a8 per-row weight scales */

struct PG {
    const uint8_t* ws; int64_t ws_pitch;           /* fp8: bf16/f32 scale grid */
    const float* as; int64_t as_pitch;
    uint16_t* y; int64_t y_pitch;
    int m, n, k;
    int as_cols, ws_cols, rblk, ws_dtype;
    int tok_tiles;
};

template <int FMT>
__global__ void __launch_bounds__(kThreads, 1)
k_tc_gemm(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
          const __grid_constant__ CUtensorMap tmS, const PG P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sc = smem + kStages * kStage;                        /* mxfp4: [kScTiles][128][32] */
    float* s_s = (float*)(sc + kScTiles * kScBytes);              /* [kFs][kTok] per-token factor of a stage */
    uint64_t* full = (uint64_t*)(s_s + kFs * kTok);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* prep = acc_empty + 2;                               /* [kSfSlots] */
    uint64_t* sc_full = prep + kSfSlots;
    uint64_t* sc_empty = sc_full + kScTiles;
    uint64_t* f_full = sc_empty + kScTiles;                       /* [kFs] factor vector written */
    uint64_t* f_empty = f_full + kFs;                             /* [kFs] ... and read by all epilogue warps */
    uint32_t* tmem_slot = (uint32_t*)(f_empty + kFs);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wt = blockIdx.x / P.tok_tiles, tt = blockIdx.x - wt * P.tok_tiles;
    const int r0 = wt * kRows, t0 = tt * kTok;
    const int nk = P.k / kStageK;
    const int ntile = (nk + 7) / 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
        for (int b = 0; b < kSfSlots; ++b) mbar_init(&prep[b], 4);
        for (int b = 0; b < kScTiles; ++b) { mbar_init(&sc_full[b], 1); mbar_init(&sc_empty[b], 4); }
        for (int b = 0; b < kFs; ++b) { mbar_init(&f_full[b], 1); mbar_init(&f_empty[b], kEpiWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 1 && warp <= 1 + kEpiWarps) {
        tc_fence_before();
        asm volatile("bar.sync 2, %0;" ::"n"(32 * (1 + kEpiWarps)) : "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = (warp >= 1 && warp <= 1 + kEpiWarps) ? *tmem_slot : 0u;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
            if (FMT == G_MXFP4) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
            auto scale_tile = [&](int tl) -> bool {
                const int r = tl % kScTiles;
                if (!mbar_wait(&sc_empty[r], ((tl / kScTiles) & 1) ^ 1, 41)) return false;
                mbar_expect_tx(&sc_full[r], (uint32_t)kScBytes);
                tma_load_2d(sc + r * kScBytes, &tmS, tl * 32, r0, &sc_full[r]);
                return true;
            };
            bool ok = true;
            if (FMT == G_MXFP4) { ok = scale_tile(0); if (ok && ntile > 1) ok = scale_tile(1); }
            for (int it = 0; it < nk && ok; ++it) {
                const int s = it % kStages;
                if (!mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1, 42)) break;
                uint8_t* st = smem + s * kStage;
                /* the unpacking tensor map counts the packed bytes it read */
                mbar_expect_tx(&full[s], (uint32_t)((FMT == G_MXFP4 ? kWBytes / 2 : kWBytes) + kABytes));
                tma_load_2d(st, &tmW, it * kStageK, r0, &full[s]);
                tma_load_2d(st + kWBytes, &tmA, it * kStageK, t0, &full[s]);
                if (FMT == G_MXFP4 && (it & 7) == 7 && (it >> 3) + 2 < ntile) ok = scale_tile((it >> 3) + 2);
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (elect_one()) {
            /* plain kinds: a format at bit 7, b format at bit 10, N >> 3 at bit 17, M >> 4 at bit 24,
             * f32 accumulate at bit 4. Block-scaled kinds: no accumulate field, scale format ue8m0 at
             * bit 23, a_sf_id at bit 29 (which byte of the row's scale word this K=32 step uses) */
            const uint32_t idesc_f8 = (1u << 4) | ((uint32_t)(kTok >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
            const uint32_t idesc_mx = (5u << 7) | ((uint32_t)(kTok >> 3) << 17) | (1u << 23) |
                                      ((uint32_t)(kRows >> 4) << 24);
            for (int it = 0; it < nk; ++it) {
                const int s = it % kStages, ab = it & 1;
                if (FMT == G_MXFP4 && !mbar_wait(&prep[it % kSfSlots], (it / kSfSlots) & 1, 43)) break;
                if (!mbar_wait(&acc_empty[ab], ((it >> 1) & 1) ^ 1, 44)) break;
                if (!mbar_wait(&full[s], (it / kStages) & 1, 45)) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(smem + s * kStage), b0 = a0 + kWBytes;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t ad = smem_desc_sw128(a0 + k * 32), bd = smem_desc_sw128(b0 + k * 32);
                    if (FMT == G_MXFP4)
                        umma_mxf8(tmem_base + ab * kTok, ad, bd, idesc_mx | ((uint32_t)k << 29),
                                  tmem_base + kSfBase + (it % kSfSlots) * 4, tmem_base + kSfbCol, k > 0 ? 1u : 0u);
                    else
                        umma_f8f6f4(tmem_base + ab * kTok, ad, bd, idesc_f8, k > 0 ? 1u : 0u);
                }
                umma_commit(&empty[s]);
                umma_commit(&acc_full[ab]);
            }
        }
    } else if (warp == 2 + kEpiWarps) {
        /* ---------------- scale warp: the per-token factor of every stage ----------------
         * factor[t] = sa[t, g] (times the tile's weight scale on the fp8 block grid). Lane l owns
         * tokens l, l+32, ...; values are fetched eight stages ahead (two blocks of four) so that no
         * stage waits on a global load. */
        constexpr bool block_grid = FMT == G_FP8;
        constexpr int TPL = (kTok + 31) / 32;                          /* tokens per lane: 6 */
        constexpr int BLK = 4;                                         /* stages per prefetch block */
        float cur[TPL][BLK], nxt[TPL][BLK], wcur[BLK], wnxt[BLK];
        const int n128 = nk;
        const float* pt[TPL];
#pragma unroll
        for (int i = 0; i < TPL; ++i) {
            const int tl = lane + 32 * i, t = t0 + tl;
            pt[i] = (tl < kTok && t < P.m) ? P.as + (int64_t)t * P.as_pitch : nullptr;
        }
        const bool vec = P.as_cols == n128 && (P.as_pitch & 3) == 0 && (((uintptr_t)P.as) & 15) == 0;
        const int64_t wrow = (int64_t)(r0 / kRows) * P.ws_pitch;
        auto load_block = [&](int b, float (*f)[BLK], float* w) {
            const bool whole = BLK * b + BLK <= nk;
#pragma unroll
            for (int j = 0; j < BLK; ++j) {
                const int x = BLK * b + j;
                w[j] = (block_grid && x < nk) ? ld_scale(P.ws, wrow + (P.ws_cols == n128 ? x : scale_col(x, P.ws_cols, n128)), P.ws_dtype) : 1.0f;
            }
#pragma unroll
            for (int i = 0; i < TPL; ++i) {
                if (pt[i] == nullptr || BLK * b >= nk) {
#pragma unroll
                    for (int j = 0; j < BLK; ++j) f[i][j] = 0.0f;
                } else if (vec && whole) {
                    const float4 v = __ldg((const float4*)(pt[i] + BLK * b));
                    f[i][0] = v.x; f[i][1] = v.y; f[i][2] = v.z; f[i][3] = v.w;
                } else {
#pragma unroll
                    for (int j = 0; j < BLK; ++j) {
                        const int x = BLK * b + j;
                        f[i][j] = x < nk ? __ldg(pt[i] + scale_col(x, P.as_cols, n128)) : 0.0f;
                    }
                }
            }
        };
        /* two blocks (eight stages) are in flight ahead of the one being handed out */
        float nx2[TPL][BLK], wnx2[BLK];
        load_block(0, cur, wcur);
        load_block(1, nxt, wnxt);
        for (int b4 = 0; b4 * BLK < nk; ++b4) {
            load_block(b4 + 2, nx2, wnx2);
#pragma unroll
            for (int j = 0; j < BLK; ++j) {
                const int it = b4 * BLK + j;
                if (it >= nk) break;
                const int sl = it % kFs;
                if (!mbar_wait(&f_empty[sl], ((it / kFs) & 1) ^ 1, 48)) { alive = false; break; }
#pragma unroll
                for (int i = 0; i < TPL; ++i)
                    if (lane + 32 * i < kTok) s_s[sl * kTok + lane + 32 * i] = block_grid ? cur[i][j] * wcur[j] : cur[i][j];
                __syncwarp();
                if (lane == 0) mbar_arrive(&f_full[sl]);
            }
            if (!alive) break;
#pragma unroll
            for (int j = 0; j < BLK; ++j) {
                wcur[j] = wnxt[j]; wnxt[j] = wnx2[j];
#pragma unroll
                for (int i = 0; i < TPL; ++i) { cur[i][j] = nxt[i][j]; nxt[i][j] = nx2[i][j]; }
            }
        }
    } else {
        /* ---------------- epilogue: thread = weight row, warp part = token third ---------------- */
        const int q = warp & 3, half = (warp - 2) >> 2;
        const int row = r0 + q * 32 + lane;
        const int rowc = min(row, P.n - 1);
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int n128 = nk;
        float acc[kHalf];
#pragma unroll
        for (int j = 0; j < kHalf; ++j) acc[j] = 0.0f;
        constexpr bool row_grid = FMT == G_FP8_ROW;
        const int64_t srow = (int64_t)rowc * P.ws_pitch;

        if (FMT == G_MXFP4 && half == 0) {
            /* the token-side scale factors are 2^0 everywhere */
#pragma unroll
            for (int c = 0; c < 8; ++c) tmem_st1(tlane + kSfbCol + c, 0x7f7f7f7fu);
        }
        /* mxfp4: this row's four E8M0 bytes of stage x go to tensor memory (warps of half 0 only) */
        auto prepare = [&](int x) -> bool {
            const int r = (x >> 3) % kScTiles, sl = x % kSfSlots;
            if ((x & 7) == 0 && !mbar_wait(&sc_full[r], ((x >> 3) / kScTiles) & 1, 46)) return false;
            const uint32_t sw = *(const uint32_t*)(sc + r * kScBytes + (q * 32 + lane) * 32 + (x & 7) * 4);
            /* the slot was last read by the MMAs of stage x - kSfSlots: their accumulator has been drained */
            tmem_st1(tlane + kSfBase + sl * 4 + q, sw);
            if ((x & 7) == 7 || x == nk - 1) { __syncwarp(); if (lane == 0) mbar_arrive(&sc_empty[r]); }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&prep[sl]);
            return true;
        };
        if (FMT == G_MXFP4 && half == 0) {
            alive = prepare(0);
            if (alive && nk > 1) alive = prepare(1);
        }
        static_assert(kHalf % 16 == 0, "the drain walks 16 columns at a time");
        float sb_next = row_grid ? ld_scale(P.ws, srow + scale_col(0, P.ws_cols, n128), P.ws_dtype) : 1.0f;
#pragma unroll 1
        for (int it = 0; it < nk && alive; ++it) {
            const int ab = it & 1, sl = it % kFs;
            const float sb = sb_next;
            if (row_grid && it + 1 < nk) sb_next = ld_scale(P.ws, srow + scale_col(it + 1, P.ws_cols, n128), P.ws_dtype);
            if (FMT == G_MXFP4 && half == 0 && it + 2 < nk) { alive = prepare(it + 2); if (!alive) break; }
            if (!mbar_wait(&f_full[sl], (it / kFs) & 1, 49)) { alive = false; break; }
            if (!mbar_wait(&acc_full[ab], (it >> 1) & 1, 47)) { alive = false; break; }
            tc_fence_after();
            const float* sf = s_s + sl * kTok + half * kHalf;
            const uint32_t ta = tlane + ab * kTok + half * kHalf;
            /* the next 16 columns' TMEM load is in flight while these are folded into the sums */
            float c[2][16];
            tmem_ld16(ta, c[0]);
#pragma unroll
            for (int ch = 0; ch < kHalf / 16; ++ch) {
                tmem_ld_wait();
                tmem_pin16(c[ch & 1]);
                if (ch + 1 < kHalf / 16) tmem_ld16(ta + (ch + 1) * 16, c[(ch + 1) & 1]);
                else {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ab]);
                }
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                    const float4 f = *(const float4*)(sf + ch * 16 + j4 * 4);
                    float* a4 = acc + ch * 16 + j4 * 4;
                    const float* c4 = c[ch & 1] + j4 * 4;
                    if (row_grid) {
                        a4[0] += (c4[0] * f.x) * sb; a4[1] += (c4[1] * f.y) * sb;
                        a4[2] += (c4[2] * f.z) * sb; a4[3] += (c4[3] * f.w) * sb;
                    } else {
                        a4[0] = fmaf(c4[0], f.x, a4[0]); a4[1] = fmaf(c4[1], f.y, a4[1]);
                        a4[2] = fmaf(c4[2], f.z, a4[2]); a4[3] = fmaf(c4[3], f.w, a4[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&f_empty[sl]);
        }
        if (alive && row < P.n) {
#pragma unroll
            for (int j = 0; j < kHalf; ++j) {
                const int t = t0 + half * kHalf + j;
                if (t < P.m) P.y[(int64_t)t * P.y_pitch + row] = f32_to_bf16(acc[j]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

bool al(const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; }

template <int FMT>
int launch(const CUtensorMap* tw, const CUtensorMap* ta, const CUtensorMap* ts, PG P, cudaStream_t st) {
    const size_t smem = 1024 + (size_t)kStages * kStage + kScTiles * kScBytes + kFs * kTok * sizeof(float) +
                        (2 * kStages + 4 + kSfSlots + 2 * kScTiles + 2 * kFs) * sizeof(uint64_t) + 64;
    static bool attr_set[kTcMaxDevices] = {};
    const int adev = tc_device();
    if (adev < 0) return RAD_E_DEVICE;
    if (!attr_set[adev]) {
        if (cudaFuncSetAttribute(k_tc_gemm<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RAD_E_DEVICE;
        attr_set[adev] = true;
    }
    const int wtiles = (P.n + kRows - 1) / kRows;
    P.tok_tiles = (P.m + kTok - 1) / kTok;
    count_launch();
    k_tc_gemm<FMT><<<(unsigned)(wtiles * P.tok_tiles), kThreads, smem, st>>>(*tw, *ta, *ts, P);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

} /* anonymous namespace */

bool tc_gemm_fp8a8_ok(const R3dGemmQ& p) {
    return p.m > 64 && (p.k % 128) == 0 && al(p.b, 16) && (p.b_pitch % 16) == 0 && al(p.a, 16) &&
           (p.a_pitch % 16) == 0 && (p.rblk == 1 || p.rblk == kRows) && (long long)p.n * ((p.m + kTok - 1) / kTok) < (1ll << 30) &&
           tc_have_encoder();
}
bool tc_gemm_mxfp4a8_ok(const R3dGemmQ& p) {
    return p.m > 64 && (p.k % 128) == 0 && al(p.b, 32) && (p.b_pitch % 32) == 0 && al(p.b_scale, 16) &&
           (p.bs_pitch % 16) == 0 && p.bs_cols == p.k / 32 && al(p.a, 16) && (p.a_pitch % 16) == 0 && tc_have_encoder();
}

int tc_gemm_fp8a8(const R3dGemmQ& p, cudaStream_t st) {
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows);
    const CUtensorMap* ta = tc_tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kTok);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    PG P{};
    P.ws = (const uint8_t*)p.b_scale; P.ws_pitch = p.bs_pitch;
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k;
    P.as_cols = p.as_cols; P.ws_cols = p.bs_cols; P.rblk = p.rblk; P.ws_dtype = p.bs_dtype;
    return p.rblk == kRows ? launch<G_FP8>(tw, ta, tw, P, st) : launch<G_FP8_ROW>(tw, ta, tw, P, st);
}

int tc_gemm_mxfp4a8(const R3dGemmQ& p, cudaStream_t st) {
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, kRows);
    const CUtensorMap* ta = tc_tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kTok);
    const CUtensorMap* ts = tc_tensor_map(p.b_scale, (uint64_t)(p.k / 32), (uint64_t)p.n, (uint64_t)p.bs_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows, 32u);
    if (!tw || !ta || !ts) return RAD_E_UNSUPPORTED;
    PG P{};
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k;
    P.as_cols = p.as_cols; P.ws_cols = p.bs_cols; P.rblk = 1; P.ws_dtype = RAD_E8M0;
    return launch<G_MXFP4>(tw, ta, ts, P, st);
}

int tc_gemm_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcg_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

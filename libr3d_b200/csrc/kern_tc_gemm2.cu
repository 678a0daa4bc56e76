/* kern_tc_gemm2.cu -- the prefill band (M > 64) for contracts whose scales do not change along K:
 * fp8a8 with one f32 scale per token and one scale per output channel (the per-channel / per-token
 * superset of gemm_nt_q @ fp8a8; the reference's grids change every 128 of K and stay on
 * kern_tc_gemm.cu). With constant scales the whole K sum is ONE tensor-memory accumulation and
 * the scales are two multiplies in the epilogue: y = bf16((sum_k a*b * sa[t]) * sb[n]) -- the
 * order of the oracle's per-group step (sub * sa) * sb, applied once to the whole sum.
 *
 * Shape of the kernel:
 *   - CTA pairs (a cluster of two, tcgen05 cta_group::2): one MMA instruction spans 256 weight rows
 *     (128 TMEM lanes in each CTA) x 256 tokens x 32 of K. Each CTA loads its own 128 weight rows
 *     and its own 128 tokens per stage (plain TMA loads, no multicast); the pair's tensor cores read
 *     the token tile halves from both CTAs' shared memory. Per 128 of K a CTA fetches 32 KiB for
 *     128 x 256 outputs, where a single-CTA 128 x 256 tile fetches 48 KiB: the prefill band is
 *     bound by the L2 -> SM operand stream, so this is the lever.
 *   - persistent: 74 pairs walk the tile list (token tiles fastest, so a wave shares its weight
 *     rows and the activations stay in L2); two 256-column accumulators in tensor memory: the
 *     epilogue of tile i (tcgen05.ld, two multiplies, bf16, store) overlaps the MMAs of tile i+1.
 *   - warp roles per CTA: warp 0 TMA producer, warp 1 TMEM owner (MMA issuer in the pair's leader),
 *     warps 2-5 epilogue (thread = weight row). The leader's barriers collect both CTAs' loads
 *     (the peer's TMA completes on the leader's mbarrier) and its tcgen05.commit releases the stage
 *     in both CTAs.
 * Every wait is bounded; on expiry a status word is set and the CTA drains and leaves.
 * Replaces, for these contracts, the tile kernel of src/r3d_gemm_fp8a8.hip:194-335 of libr3d.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#define R3D_TC_STATUS_WORD ::r3d::g_tcg2_status
namespace r3d { __device__ int g_tcg2_status = 0; }
#include "tc_common.cuh"

namespace r3d {

namespace {
using namespace tcdev;

constexpr int kRows = 128;                         /* weight rows per CTA (256 per pair) */
constexpr int kTokC = 128;                         /* tokens loaded per CTA */
constexpr int kTok = 2 * kTokC;                    /* tokens per pair tile = MMA N */
constexpr int kStageK = 128;
constexpr int kWBytes = kRows * kStageK;           /* 16 KiB */
constexpr int kABytes = kTokC * kStageK;           /* 16 KiB */
constexpr int kStage = kWBytes + kABytes;
constexpr int kStages = 6;
constexpr int kThreads = 32 * 6;
constexpr int kTmemCols = 512;

struct PG2 {
    const float* as; int64_t as_pitch;             /* one f32 per token */
    const uint8_t* ws; int64_t ws_pitch; int ws_dtype;   /* one scale per weight row */
    uint16_t* y; int64_t y_pitch;
    int m, n, k;
    int tok_tiles, tiles, pairs;
};

__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
/* TMA load of one CTA of a pair: the bytes land in this CTA's shared memory, the completion is
 * counted on `bar`, a shared::cluster address (the leader's barrier) */
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma2_f8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
/* arrive on a barrier (a shared::cluster address: this CTA's or the peer's) once every MMA issued so
 * far by this thread has completed */
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
/* arrive on a barrier of either CTA of the pair. What the arrival publishes lives in tensor memory and
 * is ordered by the tcgen05 fences on both sides, so the arrive itself needs no cluster-scope release
 * of generic memory (which cost about a microsecond per arrival when the scale warps did one per stage) */
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
k_tc_gemm_ws(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, const PG2 P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* sa_s = (float*)(smem + kStages * kStage);              /* [2][kTok] token scales of the tile in each accumulator */
    uint64_t* full = (uint64_t*)(sa_s + 2 * kTok);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_rank();
    const bool leader = crank == 0;
    const int pair = blockIdx.x >> 1;
    const int nk = P.k / kStageK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                    /* both CTAs' barriers are initialised and tensor memory is allocated */
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer: this CTA's half of both operand tiles ---------------- */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
            int s = 0; uint32_t ph = 0;
            for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
                const int wt = tile / P.tok_tiles, tt = tile - wt * P.tok_tiles;
                const int r0 = wt * 2 * kRows + (int)crank * kRows, t0 = tt * kTok + (int)crank * kTokC;
                for (int it = 0; it < nk; ++it) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, 62)) { alive = false; break; }
                    const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0u);
                    if (leader) mbar_expect_tx(&full[s], (uint32_t)(2 * kStage));
                    uint8_t* st = smem + s * kStage;
                    tma_load_2d_pair(st, &tmW, it * kStageK, r0, bar);
                    tma_load_2d_pair(st + kWBytes, &tmA, it * kStageK, t0, bar);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer (the pair's leader only) ---------------- */
        if (leader && elect_one()) {
            /* kind::f8f6f4: f32 accumulate at bit 4, a and b format e4m3 (0), N >> 3 at bit 17, M >> 4 at bit 24 */
            const uint32_t idesc = (1u << 4) | ((uint32_t)(kTok >> 3) << 17) | ((uint32_t)((2 * kRows) >> 4) << 24);
            int s = 0; uint32_t ph = 0;
            int ab = 0; uint32_t aph = 0;
            for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
                if (!mbar_wait(&acc_empty[ab], aph ^ 1u, 64)) { alive = false; break; }
                tc_fence_after();
                for (int it = 0; it < nk; ++it) {
                    if (!mbar_wait(&full[s], ph, 65)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smem + s * kStage), b0 = a0 + kWBytes;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma2_f8f6f4(tmem_base + ab * kTok, smem_desc_sw128(a0 + k * 32), smem_desc_sw128(b0 + k * 32),
                                     idesc, (it | k) ? 1u : 0u);
                    umma2_commit(smem_u32(&empty[s]));
                    umma2_commit(mapa_u32(smem_u32(&empty[s]), 1u));
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (!alive) break;
                umma2_commit(smem_u32(&acc_full[ab]));
                umma2_commit(mapa_u32(smem_u32(&acc_full[ab]), 1u));
                if (++ab == 2) { ab = 0; aph ^= 1u; }
            }
        }
    } else {
        /* ---------------- epilogue: thread = weight row of this CTA ---------------- */
        const int q = warp & 3;
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int et = threadIdx.x - 64;
        const uint32_t acc_empty_leader[2] = {mapa_u32(smem_u32(&acc_empty[0]), 0u), mapa_u32(smem_u32(&acc_empty[1]), 0u)};
        int ab = 0; uint32_t aph = 0;
        for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
            const int wt = tile / P.tok_tiles, tt = tile - wt * P.tok_tiles;
            const int row = wt * 2 * kRows + (int)crank * kRows + q * 32 + lane;
            const int t0 = tt * kTok;
            /* token scales of this tile; the buffer was last read two tiles ago */
            for (int i = et; i < kTok; i += 128)
                sa_s[ab * kTok + i] = t0 + i < P.m ? __ldg(P.as + (int64_t)(t0 + i) * P.as_pitch) : 0.0f;
            const float sb = row < P.n ? ld_scale(P.ws, (int64_t)row * P.ws_pitch, P.ws_dtype) : 0.0f;
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (!mbar_wait(&acc_full[ab], aph, 67)) { alive = false; break; }
            tc_fence_after();
            const uint32_t ta = tlane + ab * kTok;
            float c[2][16];
            tmem_ld16(ta, c[0]);
#pragma unroll 1
            for (int ch = 0; ch < kTok / 16; ch += 2) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    tmem_ld_wait();
                    tmem_pin16(c[h]);
                    if (ch + h + 1 < kTok / 16) tmem_ld16(ta + (ch + h + 1) * 16, c[h ^ 1]);
                    const float* sa = sa_s + ab * kTok + (ch + h) * 16;
                    if (row < P.n) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = t0 + (ch + h) * 16 + j;
                            if (t < P.m) P.y[(int64_t)t * P.y_pitch + row] = f32_to_bf16(__fmul_rn(__fmul_rn(c[h][j], sa[j]), sb));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader[ab]);
            if (++ab == 2) { ab = 0; aph ^= 1u; }
        }
    }
    /* the pair leaves together: the leader's MMAs read the peer's shared memory and both CTAs'
     * tensor memory is freed as one */
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

/* ------------------------------------------------------------------ mxfp4 weights x mxfp8 activations
 * The OCP-MX pair: e2m1 weights and e4m3 activations, each with one E8M0 scale per 32 of K. Both
 * scale sets are applied by the tensor core (kind::mxf8f6f4.block_scale, one scale byte per operand
 * row per K=32 instruction, read from tensor memory), so the whole K sum is one accumulation and the
 * epilogue only narrows to bf16. Same pair structure as above with [256 weight rows x 192 tokens]
 * tiles (two accumulators plus the scale-factor columns fill tensor memory). Four more warps per CTA
 * move the scale bytes: the weights' and the activations' E8M0 bytes arrive as TMA tiles of
 * [rows x 32 bytes] (eight stages each); per stage a scale warp stores its lane quarter's words --
 * weight row r at lane r, column r / 32; token n at lane n % 32 of every lane quarter, column n / 32
 * (every CTA of the pair holds the scales of all 192 tokens). */
constexpr int kTokMC = 96;                         /* tokens loaded per CTA */
constexpr int kTokM = 2 * kTokMC;                  /* tokens per pair tile */
constexpr int kABytesM = kTokMC * kStageK;         /* 12 KiB */
constexpr int kStageM = kWBytes + kABytesM;
constexpr int kStagesM = 6;
constexpr int kScRing = 2;
constexpr int kScW = kRows * 32, kScA = kTokM * 32;
constexpr int kScTileB = kScW + kScA;              /* 10 KiB: weight-scale tile + activation-scale tile of eight stages */
constexpr int kSfBaseM = 2 * kTokM;                /* 384: scale-factor columns behind the two accumulators */
constexpr int kSfSlot = 16;                        /* per stage: 4 columns for the weights, 6 (of 8) for the tokens */
constexpr int kThreadsM = 32 * 10;

struct PGM {
    uint16_t* y; int64_t y_pitch;
    int m, n, k;
    int tok_tiles, tiles, pairs;
};

__device__ __forceinline__ void umma2_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsM, 1)
k_tc_gemm_mx(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
             const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmE, const PGM P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sc = smem + kStagesM * kStageM;                      /* [kScRing][weights 128x32 | tokens 192x32] */
    uint64_t* full = (uint64_t*)(sc + kScRing * kScTileB);
    uint64_t* empty = full + kStagesM;
    uint64_t* prep = empty + kStagesM;                            /* scale factors of a stage are in both CTAs' tensor memory */
    uint64_t* acc_full = prep + kStagesM;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* sc_full = acc_empty + 2;
    uint64_t* sc_empty = sc_full + kScRing;
    uint32_t* tmem_slot = (uint32_t*)(sc_empty + kScRing);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_rank();
    const bool leader = crank == 0;
    const int pair = blockIdx.x >> 1;
    const int nk = P.k / kStageK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesM; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&prep[s], 8); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        for (int b = 0; b < kScRing; ++b) { mbar_init(&sc_full[b], 1); mbar_init(&sc_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmE) : "memory");
            int s = 0; uint32_t ph = 0;
            int r = 0; uint32_t rph = 0;
            for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
                const int wt = tile / P.tok_tiles, tt = tile - wt * P.tok_tiles;
                const int r0 = wt * 2 * kRows + (int)crank * kRows, tp = tt * kTokM, t0 = tp + (int)crank * kTokMC;
                for (int it = 0; it < nk; ++it) {
                    if ((it & 7) == 0) {
                        /* the scale bytes of the next eight stages: this CTA's 128 weight rows, the pair's 192 tokens */
                        if (!mbar_wait(&sc_empty[r], rph ^ 1u, 71)) { alive = false; break; }
                        mbar_expect_tx(&sc_full[r], (uint32_t)kScTileB);
                        tma_load_2d(sc + r * kScTileB, &tmS, (it >> 3) * 32, r0, &sc_full[r]);
                        tma_load_2d(sc + r * kScTileB + kScW, &tmE, (it >> 3) * 32, tp, &sc_full[r]);
                        if (++r == kScRing) { r = 0; rph ^= 1u; }
                    }
                    if (!mbar_wait(&empty[s], ph ^ 1u, 72)) { alive = false; break; }
                    const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0u);
                    /* the unpacking tensor map counts the packed bytes it read */
                    if (leader) mbar_expect_tx(&full[s], (uint32_t)(2 * (kWBytes / 2 + kABytesM)));
                    uint8_t* st = smem + s * kStageM;
                    tma_load_2d_pair(st, &tmW, it * kStageK, r0, bar);
                    tma_load_2d_pair(st + kWBytes, &tmA, it * kStageK, t0, bar);
                    if (++s == kStagesM) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer (the pair's leader only) ---------------- */
        if (leader && elect_one()) {
            /* block-scaled kinds: a format e2m1 (5) at bit 7, b format e4m3 (0), N >> 3 at bit 17, scale format
             * ue8m0 at bit 23, M >> 4 at bit 24; which byte of a row's scale word this K=32 step uses:
             * b_sf_id at bit 4, a_sf_id at bit 29 */
            const uint32_t idesc = (5u << 7) | ((uint32_t)(kTokM >> 3) << 17) | (1u << 23) | ((uint32_t)((2 * kRows) >> 4) << 24);
            int s = 0; uint32_t ph = 0;
            int ab = 0; uint32_t aph = 0;
            for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
                if (!mbar_wait(&acc_empty[ab], aph ^ 1u, 74)) { alive = false; break; }
                for (int it = 0; it < nk; ++it) {
                    if (!mbar_wait(&prep[s], ph, 73) || !mbar_wait(&full[s], ph, 75)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smem + s * kStageM), b0 = a0 + kWBytes;
                    const uint32_t sf = tmem_base + kSfBaseM + s * kSfSlot;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma2_mxf8(tmem_base + ab * kTokM, smem_desc_sw128(a0 + k * 32), smem_desc_sw128(b0 + k * 32),
                                   idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4), sf, sf + 4, (it | k) ? 1u : 0u);
                    umma2_commit(smem_u32(&empty[s]));
                    umma2_commit(mapa_u32(smem_u32(&empty[s]), 1u));
                    if (++s == kStagesM) { s = 0; ph ^= 1u; }
                }
                if (!alive) break;
                umma2_commit(smem_u32(&acc_full[ab]));
                umma2_commit(mapa_u32(smem_u32(&acc_full[ab]), 1u));
                if (++ab == 2) { ab = 0; aph ^= 1u; }
            }
        }
    } else if (warp >= 6) {
        /* ---------------- scale warps: lane quarter q of this CTA's tensor memory ---------------- */
        const int q = warp & 3;                                   /* warps 6..9 -> quarters 2, 3, 0, 1 */
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t prep_leader0 = mapa_u32(smem_u32(&prep[0]), 0u);
        int s = 0; uint32_t ph = 0;
        int r = 0; uint32_t rph = 0;
        for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
            for (int it = 0; it < nk; ++it) {
                if ((it & 7) == 0 && !mbar_wait(&sc_full[r], rph, 76)) { alive = false; break; }
                const uint8_t* tw = sc + r * kScTileB + (it & 7) * 4;
                const uint32_t ww = *(const uint32_t*)(tw + (q * 32 + lane) * 32);
                uint32_t wa[6];
#pragma unroll
                for (int c = 0; c < 6; ++c) wa[c] = *(const uint32_t*)(tw + kScW + (c * 32 + lane) * 32);
                if ((it & 7) == 7 || it == nk - 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sc_empty[r]);
                    if (++r == kScRing) { r = 0; rph ^= 1u; }
                }
                /* the slot was last read by the MMAs that also released shared-memory stage s */
                if (!mbar_wait(&empty[s], ph ^ 1u, 77)) { alive = false; break; }
                tc_fence_after();
                const uint32_t sf = tlane + kSfBaseM + s * kSfSlot;
                tmem_st1(sf + q, ww);
#pragma unroll
                for (int c = 0; c < 6; ++c) tmem_st1(sf + 4 + c, wa[c]);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(prep_leader0 + (uint32_t)(s * sizeof(uint64_t)));
                if (++s == kStagesM) { s = 0; ph ^= 1u; }
            }
        }
    } else {
        /* ---------------- epilogue: thread = weight row of this CTA ---------------- */
        const int q = warp & 3;
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t acc_empty_leader[2] = {mapa_u32(smem_u32(&acc_empty[0]), 0u), mapa_u32(smem_u32(&acc_empty[1]), 0u)};
        int ab = 0; uint32_t aph = 0;
        for (int tile = pair; tile < P.tiles && alive; tile += P.pairs) {
            const int wt = tile / P.tok_tiles, tt = tile - wt * P.tok_tiles;
            const int row = wt * 2 * kRows + (int)crank * kRows + q * 32 + lane;
            const int t0 = tt * kTokM;
            if (!mbar_wait(&acc_full[ab], aph, 78)) { alive = false; break; }
            tc_fence_after();
            const uint32_t ta = tlane + ab * kTokM;
            float c[2][16];
            tmem_ld16(ta, c[0]);
#pragma unroll 1
            for (int ch = 0; ch < kTokM / 16; ch += 2) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    tmem_ld_wait();
                    tmem_pin16(c[h]);
                    if (ch + h + 1 < kTokM / 16) tmem_ld16(ta + (ch + h + 1) * 16, c[h ^ 1]);
                    if (row < P.n) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = t0 + (ch + h) * 16 + j;
                            if (t < P.m) P.y[(int64_t)t * P.y_pitch + row] = f32_to_bf16(c[h][j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader[ab]);
            if (++ab == 2) { ab = 0; aph ^= 1u; }
        }
    }
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

/* ------------------------------------------------------------------ MMA-issue rate
 * The denominator for the prefill band's tensor-pipe fraction: one kernel, every CTA pair's operand
 * tiles resident in shared memory (filled once with hashed bytes), the pair's leader issues `iters`
 * stages of four K=32 MMAs back to back into two alternating accumulators, nothing is loaded or
 * stored in the timed part. kind 0: f8f6f4 e4m3 x e4m3, 256 x 256 per instruction; kind 1:
 * mxf8f6f4 block-scaled e2m1 x e4m3, 256 x 192, scale factors in tensor memory. */
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
k_mma_peak(const int kind, const int iters) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    const uint32_t crank = cluster_rank();
    /* four stages of operand tiles; e4m3 bytes with the exponent kept small so that no NaN code occurs */
    for (int i = threadIdx.x; i < 4 * kStage / 4; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        ((uint32_t*)smem)[i] = kind == 1 ? (h & 0x0f0f0f0fu) | ((h >> 3) & 0x30303030u) & 0x3f3f3f3fu : h & 0x3f3f3f3fu;
    }
    if (threadIdx.x == 0) {
        mbar_init(&done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (kind == 1) {
        /* scale factors 2^0 in the sixteen columns behind the accumulators, every lane */
        const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
        for (int c = 0; c < 16; ++c) tmem_st1(tlane + kSfBaseM + c, 0x7f7f7f7fu);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1 && crank == 0 && elect_one()) {
        const uint32_t idesc_f8 = (1u << 4) | ((uint32_t)(kTok >> 3) << 17) | ((uint32_t)((2 * kRows) >> 4) << 24);
        const uint32_t idesc_mx = (5u << 7) | ((uint32_t)(kTokM >> 3) << 17) | (1u << 23) | ((uint32_t)((2 * kRows) >> 4) << 24);
        for (int it = 0; it < iters; ++it) {
            const uint32_t a0 = smem_u32(smem + (it & 3) * kStage), b0 = a0 + kWBytes;
            const uint32_t d = tmem_base + (uint32_t)((it >> 3) & 1) * (kind == 1 ? kTokM : kTok);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (kind == 1)
                    umma2_mxf8(d, smem_desc_sw128(a0 + k * 32), smem_desc_sw128(b0 + k * 32),
                               idesc_mx | ((uint32_t)k << 29) | ((uint32_t)k << 4), tmem_base + kSfBaseM, tmem_base + kSfBaseM + 4,
                               (it & 7) | k ? 1u : 0u);
                else
                    umma2_f8f6f4(d, smem_desc_sw128(a0 + k * 32), smem_desc_sw128(b0 + k * 32), idesc_f8, (it & 7) | k ? 1u : 0u);
            }
        }
        umma2_commit(smem_u32(&done));
        (void)mbar_wait(&done, 0, 79);
    }
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

bool al(const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; }

} /* anonymous namespace */

/* fp8a8 with whole-K scale grids: one f32 per token, one scale per weight row */
bool tc_gemm_ws_fp8a8_ok(const R3dGemmQ& p) {
    static const bool off = [] { const char* e = getenv("R3D_NO_GEMM_WS"); return e && *e && *e != '0'; }();
    return !off && p.m > 64 && p.as_cols == 1 && p.bs_cols == 1 && p.rblk == 1 && (p.k % 128) == 0 && p.k >= 128 &&
           al(p.b, 16) && (p.b_pitch % 16) == 0 && al(p.a, 16) && (p.a_pitch % 16) == 0 &&
           (long long)((p.n + 255) / 256) * ((p.m + kTok - 1) / kTok) < (1ll << 30) && tc_have_encoder();
}

int tc_gemm_ws_fp8a8(const R3dGemmQ& p, cudaStream_t st) {
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows);
    const CUtensorMap* ta = tc_tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kTokC);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    const size_t smem = 1024 + (size_t)kStages * kStage + 2 * kTok * sizeof(float) + (2 * kStages + 4) * sizeof(uint64_t) + 64;
    static bool attr_set[kTcMaxDevices] = {};
    const int dev = tc_device();
    if (dev < 0) return RAD_E_DEVICE;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(k_tc_gemm_ws, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RAD_E_DEVICE;
        attr_set[dev] = true;
    }
    PG2 P{};
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.ws = (const uint8_t*)p.b_scale; P.ws_pitch = p.bs_pitch; P.ws_dtype = p.bs_dtype;
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k;
    P.tok_tiles = (p.m + kTok - 1) / kTok;
    P.tiles = ((p.n + 2 * kRows - 1) / (2 * kRows)) * P.tok_tiles;
    const int max_pairs = tc_sm_count() / 2;
    P.pairs = P.tiles < max_pairs ? P.tiles : max_pairs;
    count_launch();
    k_tc_gemm_ws<<<(unsigned)(2 * P.pairs), kThreads, smem, st>>>(*tw, *ta, P);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

/* mxfp4 weights x mxfp8 activations: R3dGemmQ.a_scale carries the activations' E8M0 bytes [M, K/32]
 * (as_cols = K/32, as_pitch in bytes) */
bool tc_gemm_mx_ok(const R3dGemmQ& p) {
    return p.m > 64 && (p.k % 128) == 0 && p.k >= 128 && al(p.b, 32) && (p.b_pitch % 32) == 0 &&
           al(p.b_scale, 16) && (p.bs_pitch % 16) == 0 && p.bs_cols == p.k / 32 &&
           al(p.a_scale, 16) && (p.as_pitch % 16) == 0 && p.as_cols == p.k / 32 &&
           al(p.a, 16) && (p.a_pitch % 16) == 0 &&
           (long long)((p.n + 255) / 256) * ((p.m + kTokM - 1) / kTokM) < (1ll << 30) && tc_have_encoder();
}

int tc_gemm_mx(const R3dGemmQ& p, cudaStream_t st) {
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, kRows);
    const CUtensorMap* ta = tc_tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kTokMC);
    const CUtensorMap* ts = tc_tensor_map(p.b_scale, (uint64_t)(p.k / 32), (uint64_t)p.n, (uint64_t)p.bs_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows, 32u);
    const CUtensorMap* te = tc_tensor_map(p.a_scale, (uint64_t)(p.k / 32), (uint64_t)p.m, (uint64_t)p.as_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kTokM, 32u);
    if (!tw || !ta || !ts || !te) return RAD_E_UNSUPPORTED;
    const size_t smem = 1024 + (size_t)kStagesM * kStageM + kScRing * kScTileB +
                        (3 * kStagesM + 4 + 2 * kScRing) * sizeof(uint64_t) + 64;
    static bool attr_set[kTcMaxDevices] = {};
    const int dev = tc_device();
    if (dev < 0) return RAD_E_DEVICE;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(k_tc_gemm_mx, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RAD_E_DEVICE;
        attr_set[dev] = true;
    }
    PGM P{};
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k;
    P.tok_tiles = (p.m + kTokM - 1) / kTokM;
    P.tiles = ((p.n + 2 * kRows - 1) / (2 * kRows)) * P.tok_tiles;
    const int max_pairs = tc_sm_count() / 2;
    P.pairs = P.tiles < max_pairs ? P.tiles : max_pairs;
    count_launch();
    k_tc_gemm_mx<<<(unsigned)(2 * P.pairs), kThreadsM, smem, st>>>(*tw, *ta, *ts, *te, P);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

/* One launch of the MMA-issue kernel on every CTA pair of the device; returns the FLOPs it issues
 * (the caller times the launch with events), or a negative status. */
extern "C" double r3d_b200_mma_peak(int kind, int iters, void* stream) {
    if (!device_is_sm100() || iters < 1 || (kind != 0 && kind != 1)) return -1.0;
    const size_t smem = 1024 + 4 * (size_t)kStage;
    static bool attr_set[kTcMaxDevices] = {};
    const int dev = tc_device();
    if (dev < 0) return -1.0;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(k_mma_peak, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1.0;
        attr_set[dev] = true;
    }
    const int pairs = tc_sm_count() / 2;
    count_launch();
    k_mma_peak<<<(unsigned)(2 * pairs), 128, smem, (cudaStream_t)stream>>>(kind, iters);
    if (cudaGetLastError() != cudaSuccess) return -1.0;
    return 2.0 * 256.0 * (kind == 1 ? (double)kTokM : (double)kTok) * 128.0 * (double)iters * (double)pairs;
}

int tc_gemm2_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcg2_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

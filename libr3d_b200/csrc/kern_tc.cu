/* kern_tc.cu -- the tcgen05 arm of the decode / verify bands: weight streaming with the
 * 5th-generation tensor cores doing the dequantisation.
 *
 * Shape of the problem: y[M,N] = a[M,K] . w[N,K]^T with M <= 64 tokens. The weight plane is
 * the only large operand, so the kernel is "swap-AB": 128 weight rows sit on the M axis of
 * tcgen05.mma (one TMEM lane per weight row) and the tokens, padded to 16/32/64, on its N
 * axis. Everything the CUDA cores did in the mma.sync arm disappears:
 *   - TMA tensor maps bring a [128 rows x 128 K] weight tile per stage straight into the
 *     128-byte-swizzled shared layout the MMA descriptor wants. For mxfp4a8 the tensor map
 *     type CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B unpacks the e2m1 nibbles on the way in (HBM
 *     traffic stays 4 bits per weight) and kind::f8f6f4 decodes them in the tensor core:
 *     no conversion instruction is executed anywhere.
 *   - The activation tile [tokens x 128 K] comes the same way (rows past M are zero-filled
 *     by the TMA unit).
 *   - One elected thread issues four K=32 MMAs per stage; accumulators live in TMEM, double
 *     buffered so the next stage's MMAs run while the epilogue drains this one.
 *   - Four epilogue warps (128 threads = 128 weight rows) read the f32 partials with
 *     tcgen05.ld and apply the scale groups in registers, in the reference's flush order:
 *       fp8a8    acc += (sub128 * sa[m,g]) * sb[row,g]                 (one partial per stage)
 *       mxfp4a8  acc += (sum_j sub32_j * 2^(x_j-127)) * sa[m,g]: the E8M0 group scales are applied
 *                by the tensor core (kind::mxf8f6f4.block_scale, one scale per K=32 MMA) from
 *                tensor memory, where the epilogue warps put each row's four bytes per stage
 * Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 epilogue.
 *
 * Every mbarrier wait is bounded (~1 s of clock64); on expiry a status word is set
 * (r3d_b200_stream_status() reports it) and the CTA drains, frees its TMEM and leaves
 * without storing.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>
#include <vector>
#define R3D_TC_STATUS_WORD ::r3d::g_tc_status
namespace r3d { __device__ int g_tc_status = 0; }   /* nonzero = code of the bounded wait that expired */
#include "tc_common.cuh"
#include "push.cuh"

namespace r3d {

int tc_mxf4_status();                               /* kern_tc_mxf4.cu's status word */
int tc_gemm_status();                               /* kern_tc_gemm.cu's status word */

namespace {

constexpr int kTcThreads = 192;
constexpr int kTileRows = 128;
constexpr int kStageK = 128;                       /* K elements (= smem bytes per row) per stage */
constexpr int kABytes = kTileRows * kStageK;       /* 16 KiB */

enum { TC_FP8 = 0, TC_MXFP4 = 1 };

struct TcParams {
    const uint8_t* ws; int64_t ws_pitch;           /* weight scales: bf16/f32 grid or E8M0 bytes */
    const float* as; int64_t as_pitch;
    void* y; int64_t y_pitch; int y_dtype;
    int m, mlive, n, k;                            /* m: activation rows staged; mlive: rows stored */
    int as_cols, ws_cols, rblk, ws_dtype;
    int ksplit;                                    /* CTAs per cluster = K shares per row tile */
    PushCfg push;                                  /* world > 0: store into every rank's gathered buffer */
    /* gemm_nt_q_gated: the weight is [2 n_half, K], gate rows first. A cluster of two CTAs takes gate tile g
     * and up tile g over the whole K; the gate CTA closes the call with the gated quantiser
     * (src/r3d_gemm_fp8a8.hip:700-825 of libr3d) instead of storing y */
    int gated, gsilu, gob_dtype;
    uint8_t* gq; int64_t gq_pitch;                 /* e4m3 codes [M, n_half] */
    float* gs; int64_t gs_pitch;                   /* f32 scale [M, n_half / 128] */
    void* gob; int64_t gob_pitch;                  /* optional gated product, bf16 or f32 */
};

using namespace tcdev;

/* NTOK: tokens on the MMA's N axis (16, 32 or 64; rows past M are zero). ML: tokens the
 * epilogue actually reads and stores (M rounded up to 1, 2, 4, 8, 16, ...): the TMEM columns
 * of padding tokens are never touched. The CTAs of a cluster split K between them and the
 * leader adds the partial sums through distributed shared memory, in rank order. */
template <int FMT, int NTOK, int ML, int kTcStages, int LG, int GATED>
__global__ void __launch_bounds__(kTcThreads, (GATED && ML <= 32) ? 2 : 1)
k_tc_decode(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
            const TcParams P) {
    constexpr int kBBytes = NTOK * kStageK;
    constexpr int kStage = kABytes + kBBytes;
    constexpr int kAccCols = NTOK;                                 /* per buffer */
    constexpr int kBufs = 4;                                       /* accumulator ring in TMEM */
    /* mxfp4a8: after the accumulators, four scale-factor columns per smem stage (one 32-bit word
     * per weight row, in column base + lane quarter) and eight columns of token-side factors */
    constexpr int kSfBase = kBufs * kAccCols;
    constexpr int kSfbCol = kSfBase + kTcStages * 4;
    constexpr int kNeedCols = FMT == TC_MXFP4 ? kSfbCol + 8 : kBufs * kAccCols;
    constexpr int kTmemCols = kNeedCols <= 32 ? 32 : (kNeedCols <= 64 ? 64 : (kNeedCols <= 128 ? 128 : 256));
    static_assert(kNeedCols <= 256, "TMEM columns");
    constexpr int LEAD = kTcStages >= 4 ? 3 : 2;                   /* mxfp4a8: scale words go to TMEM this many stages ahead */

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + kTcStages * kStage);
    uint64_t* empty = full + kTcStages;
    uint64_t* acc_full = empty + kTcStages;
    uint64_t* acc_empty = acc_full + 4;
    uint64_t* prep = acc_empty + 4;                                 /* [kTcStages] mxfp4a8: scale factors are in TMEM */
    uint32_t* tmem_slot = (uint32_t*)(prep + kTcStages);
    float* as_s = (float*)(tmem_slot + 4);                          /* [n128][NTOK] */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ks = P.ksplit;
    const int crank = ks > 1 ? (int)cluster_rank() : 0;
    const int n128 = P.k / kStageK;
    /* gated: cluster rank 0 = gate tile, rank 1 = the up tile n_half rows below, both over all of K */
    const int r0 = GATED ? (int)(blockIdx.x / 2) * kTileRows + (crank ? P.n / 2 : 0) : (blockIdx.x / ks) * kTileRows;
    const int it0 = GATED ? 0 : (int)((int64_t)n128 * crank / ks);    /* this CTA's K stages */
    const int nk = GATED ? n128 : (int)((int64_t)n128 * (crank + 1) / ks) - it0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&prep[s], 4); }
        for (int b = 0; b < kBufs; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();                       /* barriers are initialised: the producer may start */
    dep_launch();                          /* the next kernel of the stream may begin its own prologue */
    /* The rest of the set-up overlaps the first weight loads: the MMA warp owns the TMEM
     * allocation, the epilogue warps stage the activation scales (rows past M read as 0);
     * the five warps then meet on a named barrier, which the producer does not wait for. */
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else if (warp >= 2) {
        dep_wait();                        /* activation scales are the previous kernel's output */
        /* This staging sits between the previous kernel's end and this kernel's first flush: thread = 128-K
         * group, the live tokens' scales along their rows (coalesced), eight loads in flight a thread (one
         * load a turn of a loop cost a microsecond on 4096 x 4096 and 3.6 us at K = 13824, sixteen tokens). */
        const int et = threadIdx.x - 64;
        const int gend = it0 + nk;                     /* this CTA's K share */
        /* few groups (a K share of a cluster, a short K): the 128 threads split the tokens between them too */
        const int parts = nk <= 32 ? 4 : nk <= 64 ? 2 : 1;
        const int lanes = 128 / parts, part = et / lanes, gl = et - part * lanes;
        const int tpp = NTOK / parts;                  /* tokens a part: NTOK is 16, 32 or 64 */
        for (int g0 = it0; g0 < gend; g0 += lanes) {
            const int g = g0 + gl;
            const int col = g < gend ? scale_col(g, P.as_cols, n128) : 0;
            for (int tb = 0; tb < tpp; tb += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int t = part * tpp + tb + u;
                    v[u] = (g < gend && tb + u < tpp && t < P.m) ? __ldg(P.as + (int64_t)t * P.as_pitch + col) : 0.0f;
                }
                if (g < gend) {
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (tb + u < tpp) as_s[g * NTOK + part * tpp + tb + u] = v[u];
                }
            }
        }
    }
    if (warp >= 1) {
        tc_fence_before();
        asm volatile("bar.sync 2, 160;" ::: "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = warp >= 1 ? *tmem_slot : 0u;

    const int q = warp & 3;                                    /* TMEM lane quarter of an epilogue warp */
    const int row = r0 + q * 32 + lane;
    float acc[ML];
#pragma unroll
    for (int t = 0; t < ML; ++t) acc[t] = 0.0f;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
            /* Weights depend on nothing that runs before this kernel: the first ring of weight
             * tiles is requested at once. Activation tiles are the previous kernel's output and
             * are requested after dep_wait(); they complete the same stage barriers. */
            const int first = nk < kTcStages ? nk : kTcStages;
            for (int it = 0; it < nk; ++it) {
                const int s = it % kTcStages;
                if (!mbar_wait(&empty[s], ((it / kTcStages) & 1) ^ 1, 11)) break;
                uint8_t* st = smem + s * kStage;
                /* the unpacking tensor map counts the packed bytes it read, not the padded
                 * bytes it wrote */
                mbar_expect_tx(&full[s], (uint32_t)((FMT == TC_MXFP4 ? kABytes / 2 : kABytes) + kBBytes));
                tma_load_2d(st, &tmW, (it0 + it) * kStageK, r0, &full[s]);
                if (it == first - 1) {
                    dep_wait();
                    for (int j = 0; j < first; ++j)
                        tma_load_2d(smem + j * kStage + kABytes, &tmA, (it0 + j) * kStageK, 0, &full[j]);
                } else if (it >= first) {
                    tma_load_2d(st + kABytes, &tmA, (it0 + it) * kStageK, 0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (elect_one()) {
            /* plain kinds: f32 accumulate at bit 4, a format at bit 7, N >> 3 at bit 17, M >> 4 at bit
             * 24. Block-scaled kinds: a format e2m1 (5) at bit 7, scale format ue8m0 at bit 23,
             * a_sf_id (which byte of the row's scale word this K=32 step uses) at bit 29 */
            const uint32_t idesc = FMT == TC_MXFP4
                ? ((5u << 7) | ((uint32_t)(NTOK >> 3) << 17) | (1u << 23) | ((uint32_t)(kTileRows >> 4) << 24))
                : ((1u << 4) | ((uint32_t)(NTOK >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24));
            for (int it = 0; it < nk; ++it) {
                const int s = it % kTcStages, buf = it % kBufs;
                if (FMT == TC_MXFP4 && !mbar_wait(&prep[s], (it / kTcStages) & 1, 15)) break;
                if (!mbar_wait(&acc_empty[buf], ((it / kBufs) & 1) ^ 1, 12)) break;
                if (!mbar_wait(&full[s], (it / kTcStages) & 1, 13)) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(smem + s * kStage), b0 = a0 + kABytes;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t ad = smem_desc_sw128(a0 + k * 32), bd = smem_desc_sw128(b0 + k * 32);
                    if (FMT == TC_MXFP4)
                        umma_mxf8(tmem_base + buf * kAccCols, ad, bd, idesc | ((uint32_t)k << 29),
                                  tmem_base + kSfBase + s * 4, tmem_base + kSfbCol, k > 0 ? 1u : 0u);
                    else
                        umma_f8f6f4(tmem_base + buf * kAccCols, ad, bd, idesc, k > 0 ? 1u : 0u);
                }
                umma_commit(&empty[s]);          /* smem stage reusable once these MMAs retire */
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        /* ---------------- epilogue: thread = weight row ---------------- */
        const int rowc = min(row, P.n - 1);
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int64_t srow = (FMT == TC_FP8) ? (int64_t)(P.rblk > 1 ? rowc / P.rblk : rowc) * P.ws_pitch
                                             : (int64_t)rowc * P.ws_pitch;
        /* Weight scales of this row, fetched eight stages ahead of their use: the loads are
         * DRAM-latency long and sit on the epilogue's serial path otherwise. */
        constexpr int PF = 8;
        float sbn[PF];
        uint32_t swn[PF];
        auto fetch = [&](int blk) {
#pragma unroll
            for (int j = 0; j < PF; ++j) {
                const int it = blk * PF + j;
                if (FMT == TC_FP8)
                    sbn[j] = it < nk ? ld_scale(P.ws, srow + scale_col((it0 + it), P.ws_cols, n128), P.ws_dtype) : 0.0f;
                else
                    swn[j] = it < nk ? __ldg((const uint32_t*)(P.ws + srow + (it0 + it) * 4)) : 0u;
            }
        };
        fetch(0);
        /* mxfp4a8: stage x's scale word goes to tensor memory LEAD stages ahead of its MMAs; the
         * column set belongs to the smem stage slot, free once the MMAs of stage x - stages retired */
        auto prepare = [&](int x, uint32_t sw) -> bool {
            const int s = x % kTcStages;
            if (!mbar_wait(&empty[s], ((x / kTcStages) & 1) ^ 1, 16)) return false;
            tc_fence_after();
            tmem_st1(tlane + kSfBase + s * 4 + q, sw);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&prep[s]);
            return true;
        };
        if (FMT == TC_MXFP4) {
            /* the token-side scale factors are 2^0 everywhere */
#pragma unroll
            for (int c = 0; c < 8; ++c) tmem_st1(tlane + kSfbCol + c, 0x7f7f7f7fu);
#pragma unroll
            for (int x = 0; x < LEAD; ++x)
                if (x < nk && alive) alive = prepare(x, swn[x]);
        }
        for (int blk = 0; blk * PF < nk && alive; ++blk) {
            float sbc[PF];
            uint32_t swc[PF];
#pragma unroll
            for (int j = 0; j < PF; ++j) { sbc[j] = sbn[j]; swc[j] = swn[j]; }
            fetch(blk + 1);
#pragma unroll
            for (int j8 = 0; j8 < PF; ++j8) {
                const int it = blk * PF + j8;
                if (it >= nk) break;
                const int buf = it % kBufs;
                if (FMT == TC_MXFP4 && it + LEAD < nk) {
                    alive = prepare(it + LEAD, j8 + LEAD < PF ? swc[(j8 + LEAD) % PF] : swn[(j8 + LEAD) % PF]);
                    if (!alive) break;
                }
                if (!mbar_wait(&acc_full[buf], (it / kBufs) & 1, 14)) { alive = false; break; }
                tc_fence_after();
                const float* sa = as_s + (it0 + it) * NTOK;
                if (FMT == TC_FP8) {
                    const float sb = sbc[j8];
                    float c[ML];
                    tmem_ld<ML>(tlane + buf * kAccCols, c);
                    tmem_ld_wait();
                    tmem_pin<ML>(c);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
#pragma unroll
                    for (int t = 0; t < ML; ++t) {
                        /* logits: the piece scale is a power of two, so scaling by it last costs
                         * no rounding and cannot overflow before the weight scale shrinks c */
                        if (LG) acc[t] += (c[t] * sb) * sa[t];
                        else acc[t] += (c[t] * sa[t]) * sb;
                    }
                } else {
                    float c[ML];
                    tmem_ld<ML>(tlane + buf * kAccCols, c);
                    tmem_ld_wait();
                    tmem_pin<ML>(c);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
#pragma unroll
                    for (int t = 0; t < ML; ++t) acc[t] += c[t] * sa[t];
                }
            }
        }
        if (ks > 1 && (crank != 0 || GATED)) {
            /* every stage of this CTA has been consumed: the stage ring is free to carry the
             * partial sums to the leader (gated: each CTA's bf16-rounded outputs to its partner) */
            float* red = (float*)smem;
#pragma unroll
            for (int t = 0; t < ML; ++t)
                red[t * kTileRows + q * 32 + lane] = !alive ? __int_as_float(0x7fc00000)
                                                     : GATED ? bf16_to_f32(f32_to_bf16(acc[t])) : acc[t];
        }
    }

    if (ks > 1) {
        cluster_sync_all();                                   /* partial sums are in place */
        if (!GATED && warp >= 2 && crank == 0) {
            const float* red = (const float*)smem;
            int r = 1;
            if (ML <= 16) {
                /* up to four peers' partial sums are requested together (a remote read is a few hundred
                 * nanoseconds; one peer after the other cost the small shapes most of a microsecond) and
                 * added in rank order */
                float pr[4][ML];
#pragma unroll
                for (int p = 0; p < 4; ++p)
#pragma unroll
                    for (int t = 0; t < ML; ++t)
                        pr[p][t] = p + 1 < ks ? ld_peer_f32(red + t * kTileRows + q * 32 + lane, (uint32_t)(p + 1)) : 0.0f;
#pragma unroll
                for (int p = 0; p < 4; ++p)
                    if (p + 1 < ks) {
#pragma unroll
                        for (int t = 0; t < ML; ++t) acc[t] += pr[p][t];
                    }
                r = 5;
            }
            for (; r < ks; ++r)
#pragma unroll
                for (int t = 0; t < ML; ++t) acc[t] += ld_peer_f32(red + t * kTileRows + q * 32 + lane, (uint32_t)r);
        }
        if (GATED && warp >= 2) {
            /* The gated quantiser over this pair's 128 columns of n (one quantiser group), every statement as
             * k_gated_quant_fp8 has it: the band's outputs rounded to bf16, h = bf16((silu ? gt*sg : sg) * up)
             * with sg through a double-precision exp, the group's amax (NaN never wins), scale = amax / 448
             * (1 when amax = 0), saturating RTNE e4m3 codes of h / scale. Thread = column of n. The two CTAs
             * share the tokens (even slots: the gate CTA, odd slots: the up CTA; each reads the other half of
             * its operands from its partner's shared memory): the exponentials are the cost of this tail. */
            const float* red = (const float*)smem;
            float* amax_s = (float*)smem + ML * kTileRows;      /* own stage ring, past the exported values */
            const int col = (int)(blockIdx.x / 2) * kTileRows + q * 32 + lane;
            float other[(ML + 1) / 2];
#pragma unroll
            for (int t = 0; t < ML; ++t)
                if ((t & 1) == crank) other[t >> 1] = ld_peer_f32(red + t * kTileRows + q * 32 + lane, (uint32_t)(crank ^ 1));
#pragma unroll
            for (int t = 0; t < ML; ++t) {
                if ((t & 1) != crank) continue;
                const float mine = bf16_to_f32(f32_to_bf16(acc[t]));
                const float gt = crank ? other[t >> 1] : mine;
                const float up = crank ? mine : other[t >> 1];
                const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-gt))));
                const float a = P.gsilu ? __fmul_rn(gt, sg) : sg;
                const float h = bf16_to_f32(f32_to_bf16(__fmul_rn(a, up)));
                acc[t] = h;
                float mx = fabsf(h);
                if (!(mx > 0.0f)) mx = 0.0f;                    /* NaN and zero start the maximum at 0 */
                for (int off = 16; off; off >>= 1) {
                    const float o = __shfl_xor_sync(0xffffffffu, mx, off);
                    if (o > mx) mx = o;
                }
                if (lane == 0) amax_s[q * ML + t] = mx;
            }
            asm volatile("bar.sync 3, 128;" ::: "memory");
            const int grp = (int)(blockIdx.x / 2);
#pragma unroll
            for (int t = 0; t < ML; ++t) {
                if ((t & 1) != crank || t >= P.mlive || !alive) continue;
                float r = amax_s[t];
                for (int w = 1; w < 4; ++w) if (amax_s[w * ML + t] > r) r = amax_s[w * ML + t];
                const float sc = r > 0.0f ? __fmul_rn(r, 1.0f / 448.0f) : 1.0f;
                if (q == 0 && lane == 0) P.gs[(int64_t)t * P.gs_pitch + grp] = sc;
                const float inv = __fdiv_rn(1.0f, sc);
                const float h = acc[t];
                if (P.gob) {
                    if (P.gob_dtype == RAD_F32) ((float*)P.gob)[(int64_t)t * P.gob_pitch + col] = h;
                    else ((uint16_t*)P.gob)[(int64_t)t * P.gob_pitch + col] = f32_to_bf16(h);
                }
                float c = __fmul_rn(h, inv);
                if (c > 448.0f) c = 448.0f;
                if (c < -448.0f) c = -448.0f;
                P.gq[(int64_t)t * P.gq_pitch + col] = f32_to_e4m3(c);
            }
        }
    }
    if (!GATED && warp >= 2 && crank == 0 && alive && row < P.n) {
        if (LG) {
            /* activation rows [0, ML/2) carry the leading piece of each token and rows
             * [ML/2, ML) the residual piece: their sums are the token's logit */
#pragma unroll
            for (int t = 0; t < ML / 2; ++t) {
                if (t >= P.mlive) break;
                const float v = acc[t] + acc[t + ML / 2];
                if (P.y_dtype == RAD_F32) {
                    if (P.push.world) push_store<float>(P.push, t, row, v);
                    else ((float*)P.y)[(int64_t)t * P.y_pitch + row] = v;
                } else {
                    if (P.push.world) push_store<uint16_t>(P.push, t, row, f32_to_bf16(v));
                    else ((uint16_t*)P.y)[(int64_t)t * P.y_pitch + row] = f32_to_bf16(v);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < ML; ++t) {
                if (t >= P.mlive) break;
                if (P.push.world) push_store<uint16_t>(P.push, t, row, f32_to_bf16(acc[t]));
                else ((uint16_t*)P.y)[(int64_t)t * P.y_pitch + row] = f32_to_bf16(acc[t]);
            }
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

/* ------------------------------------------------------------------ host: tensor maps */
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        (void)cudaGetLastError();
        return (EncodeTiledFn)p;
    }();
    return fn;
}

struct MapKey {
    const void* ptr; uint64_t d0, d1, pitch; int dtype; uint32_t box1, box0; int dev, promo;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && pitch == o.pitch && dtype == o.dtype &&
               box1 == o.box1 && box0 == o.box0 && dev == o.dev && promo == o.promo;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9E3779B97F4A7C15ull;
        h ^= (k.d0 + 0x632BE59BD9B4E019ull) * 0xD6E8FEB86659FD93ull;
        h ^= (k.d1 * 0xFF51AFD7ED558CCDull) ^ (k.pitch << 17) ^ ((uint64_t)k.box1 << 40) ^ ((uint64_t)k.box0 << 52) ^
             ((uint64_t)k.dtype << 8) ^ ((uint64_t)k.dev << 3) ^ (uint64_t)k.promo;
        return (size_t)(h ^ (h >> 29));
    }
};

/* Tensor maps are remembered per (device, pointer, geometry): the engine's buffers are long-lived and
 * a launch must not do driver work in steady state. Single dispatch thread, like the reference's
 * plane cache (src/r3d_gemm_mxfp4.hip:1879-1880). A lookup hands out a copy in a small ring, so the
 * maps of one launch (at most four lookups) stay valid whatever the table does in between; when the
 * table is full (activation buffers that keep moving) it is emptied and refills with what is live. */
const CUtensorMap* tensor_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                              CUtensorMapDataType dt, uint32_t box1, uint32_t box0 = 128u, int promo128 = 0) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static CUtensorMap ring[16];
    static unsigned ring_at = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    const MapKey key{ptr, d0, d1, pitch_bytes, (int)dt, box1, box0, dev, promo128};
    CUtensorMap* slot = &ring[ring_at++ & 15u];
    auto it = cache.find(key);
    if (it != cache.end()) { *slot = it->second; return slot; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return nullptr;
    const cuuint64_t dims[2] = {d0, d1};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1u, 1u};
    CUtensorMap m;
    const CUresult rc = fn(&m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           box0 == 128u ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           promo128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return nullptr;
    if (cache.size() >= 16384) cache.clear();
    cache.emplace(key, m);
    *slot = m;
    return slot;
}

int sm_count();

/* K shares per row tile (the CTAs of one cluster; never more shares than whole stages). Measured over 16
 * to 216 row tiles (M = 1..16, K = 4096..13824): the best share count keeps the grid near 190-250 CTAs
 * and never past five shares -- more CTAs than the device holds at once (two per SM) wait for a second
 * wave (tiles * shares of 298 ran up to 70 % slower), and six to eight shares cost more in the reduction
 * than they stream. 124 to 148 tiles (one CTA per SM, half the device's slots idle: the slab of a head
 * sharded eight ways) take two shares, 296 CTAs at most (measured on 148 tiles x 5120: 21.5 -> 19.7 us).
 * Splitting off the few tiles past a whole number of waves into a second grid with five shares was
 * measured and dropped (297 tiles: 41.9 -> 41.0 us; the full head 119 -> 125 us: the remainder already
 * overlaps the last wave and the next call's prefetch). */
int k_shares(int tiles, int n128, int ctas_per_sm) {
    static const int forced = [] { const char* e = getenv("R3D_TC_KSPLIT"); return e ? atoi(e) : 0; }();
    const int sms = sm_count();
    int ks = forced > 0 ? forced : (5 * sms / 3) / (tiles > 0 ? tiles : 1);
    if (forced <= 0 && ks > 5) ks = 5;
    if (forced <= 0 && ks == 1 && tiles <= sms && ctas_per_sm >= 2) ks = 2;
    if (ks > 8) ks = 8;
    if (ks > n128) ks = n128;
    return ks < 1 ? 1 : ks;
}

template <int FMT, int NTOK, int ML, int kTcStages, int LG, int GATED>
int launch_tc_s(const CUtensorMap* tw, const CUtensorMap* ta, TcParams P, cudaStream_t st) {
    const size_t smem = 1024 + (size_t)kTcStages * (kABytes + NTOK * kStageK) +
                        (3 * kTcStages + 8) * sizeof(uint64_t) + 16 +
                        (size_t)(P.k / kStageK) * NTOK * sizeof(float);
    if (smem > 220 * 1024) return RAD_E_UNSUPPORTED;
    static size_t attr_set_dev[kTcMaxDevices] = {};
    const int adev = tc_device();
    if (adev < 0) return RAD_E_DEVICE;
    size_t& attr_set = attr_set_dev[adev];
    if (smem > attr_set) {
        if (cudaFuncSetAttribute(k_tc_decode<FMT, NTOK, ML, kTcStages, LG, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return RAD_E_DEVICE;
        /* ask for the largest shared-memory carve-out so that two CTAs fit on an SM */
        (void)cudaFuncSetAttribute(k_tc_decode<FMT, NTOK, ML, kTcStages, LG, GATED>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   (int)cudaSharedmemCarveoutMaxShared);
        attr_set = smem;
    }
    const int tiles = (P.n + kTileRows - 1) / kTileRows;
    /* gated: tiles = gate tiles + up tiles, one cluster a pair */
    const int ks = GATED ? 2 : k_shares(tiles, P.k / kStageK, 2 * smem + 2048 <= 233472 ? 2 : 1);
    P.ksplit = ks;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(GATED ? tiles : tiles * ks));
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)ks; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = tc_pdl_on() ? 2 : 1;
    count_launch();
    const cudaError_t e = cudaLaunchKernelEx(&cfg, k_tc_decode<FMT, NTOK, ML, kTcStages, LG, GATED>, *tw, *ta, P);
    return e == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

template <int FMT, int NTOK, int ML, int LG = 0, int GATED = 0>
int launch_tc(const CUtensorMap* tw, const CUtensorMap* ta, TcParams P, cudaStream_t st) {
    /* the deepest ring that still lets two CTAs share an SM (233472 bytes of shared memory,
     * 1 KiB of it reserved per CTA): two CTAs' streams together are what saturates HBM */
    const size_t fixed = 1024 + (3 * 6 + 8) * sizeof(uint64_t) + 16 + (size_t)(P.k / kStageK) * NTOK * sizeof(float);
    const size_t stage = kABytes + NTOK * kStageK;
    const size_t half = 233472 / 2 - 1024;
    if (fixed + 6 * stage <= half) return launch_tc_s<FMT, NTOK, ML, 6, LG, GATED>(tw, ta, P, st);
    /* 32 token columns: six stages no longer fit twice; five do (measured on the head at sixteen tokens:
     * 142.6 -> 138.1 us against four; the mxfp4 form lost 5 us with five and keeps four) */
    if (FMT == TC_FP8 && NTOK == 32 && fixed + 5 * stage <= half) return launch_tc_s<FMT, NTOK, ML, 5, LG, GATED>(tw, ta, P, st);
    if (fixed + 4 * stage <= half) return launch_tc_s<FMT, NTOK, ML, 4, LG, GATED>(tw, ta, P, st);
    if (fixed + 3 * stage <= half) return launch_tc_s<FMT, NTOK, ML, 3, LG, GATED>(tw, ta, P, st);
    return launch_tc_s<FMT, NTOK, ML, 6, LG, GATED>(tw, ta, P, st);          /* one CTA per SM */
}

int sm_count() {
    static int per_dev[kTcMaxDevices] = {};
    const int dev = tc_device();
    if (dev < 0) return 148;
    if (!per_dev[dev]) {
        int v = 148;
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        per_dev[dev] = v > 0 ? v : 148;
    }
    return per_dev[dev];
}


/* ------------------------------------------------------------------ logits: activation split
 * The LM head multiplies bf16 activations (not quantised ones) with e4m3 codes. tcgen05 has no
 * mixed bf16 x e4m3 kind, so each bf16 activation is written as the exact sum of two e4m3
 * numbers on a per-(token, 128-column block) power-of-two grid:
 *     x = s * (hi + lo / 16),   s = 2^(floor(log2(amax)) - 7)   (amax of the block -> [128, 256))
 * hi = RNE_e4m3(x / s) keeps the leading four significant bits; the residual x/s - hi is a
 * multiple of 2^(e-7) no larger than 2^(e-4) (e = exponent of x/s), so 16 * residual has at
 * most four significant bits and is an e4m3 number as long as e >= -6. Elements more than
 * 2^13 below their block's amax lose bits below amax * 2^-22; every other element is exact.
 * hi rows and lo rows ride the MMA's N axis as separate "tokens" with scales s and s/16. */
constexpr int kLgMaxTok = 32;                      /* tokens per pass (two piece rows each) */
constexpr int kLgMaxK = 16384;
__device__ __align__(256) uint8_t g_lg_pieces[2 * kLgMaxTok * kLgMaxK];
__device__ __align__(256) float g_lg_scale[2 * kLgMaxTok * (kLgMaxK / 128)];

/* one warp per (token slot t < mp, 128-column block g); slots t >= m are written as zeros */
__global__ void __launch_bounds__(128)
k_lg_split(const uint16_t* __restrict__ x, int64_t x_pitch, int m, int mp, int k,
           uint8_t* __restrict__ pieces, float* __restrict__ scale) {
    dep_launch();
    dep_wait();                    /* x is the previous kernel's output; the previous reader of the
                                      piece rows must have finished */
    const int n128 = k / 128;
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= mp * n128) return;
    const int t = w / n128, g = w - t * n128;
    uint8_t* hi = pieces + (int64_t)t * k + g * 128 + lane * 4;
    uint8_t* lo = pieces + (int64_t)(mp + t) * k + g * 128 + lane * 4;
    if (t >= m) {
        *(uint32_t*)hi = 0u; *(uint32_t*)lo = 0u;
        if (lane == 0) { scale[t * n128 + g] = 0.0f; scale[(mp + t) * n128 + g] = 0.0f; }
        return;
    }
    const uint2 raw = __ldg((const uint2*)(x + (int64_t)t * x_pitch + g * 128 + lane * 4));
    float v[4] = {bf16_to_f32((uint16_t)(raw.x & 0xffff)), bf16_to_f32((uint16_t)(raw.x >> 16)),
                  bf16_to_f32((uint16_t)(raw.y & 0xffff)), bf16_to_f32((uint16_t)(raw.y >> 16))};
    float amax = 0.0f;
    bool finite = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = fabsf(v[i]);
        if (a <= 3.4028234e38f) amax = fmaxf(amax, a); else finite = false;   /* false for inf, NaN */
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int e = 0;
    if (amax > 0.0f) { (void)frexpf(amax, &e); e -= 1; }        /* amax = f * 2^e, f in [1, 2) */
    const int sh = amax > 0.0f ? e - 7 : 0;
    uint32_t ph = 0, pl = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint8_t ch, cl;
        if (!(fabsf(v[i]) <= 3.4028234e38f)) { ch = 0x7f; cl = 0; }   /* inf, NaN -> e4m3 NaN */
        else {
            const float xs = scalbnf(v[i], -sh);
            ch = f32_to_e4m3(xs);
            cl = f32_to_e4m3((xs - e4m3_to_f32(ch)) * 16.0f);
        }
        ph |= (uint32_t)ch << (8 * i); pl |= (uint32_t)cl << (8 * i);
    }
    (void)finite;
    *(uint32_t*)hi = ph; *(uint32_t*)lo = pl;
    if (lane == 0) {
        scale[t * n128 + g] = scalbnf(1.0f, sh);
        scale[(mp + t) * n128 + g] = scalbnf(1.0f, sh - 4);
    }
}

struct LgScratch { uint8_t* pieces; float* scale; };
/* address of the static scratch on the current device, looked up once per device */
bool lg_scratch(LgScratch* out) {
    static LgScratch per_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!per_dev[dev].pieces) {
        void *p = nullptr, *q = nullptr;
        if (cudaGetSymbolAddress(&p, g_lg_pieces) != cudaSuccess ||
            cudaGetSymbolAddress(&q, g_lg_scale) != cudaSuccess) { (void)cudaGetLastError(); return false; }
        per_dev[dev].pieces = (uint8_t*)p; per_dev[dev].scale = (float*)q;
    }
    *out = per_dev[dev];
    return true;
}

template <int FMT, int NTOK, int GATED = 0>
int launch_tc_ml(const CUtensorMap* tw, const CUtensorMap* ta, const TcParams& P, cudaStream_t st) {
    if (NTOK == 16) {
        if (P.m <= 1) return launch_tc<FMT, 16, 1, 0, GATED>(tw, ta, P, st);
        if (P.m <= 2) return launch_tc<FMT, 16, 2, 0, GATED>(tw, ta, P, st);
        if (P.m <= 4) return launch_tc<FMT, 16, 4, 0, GATED>(tw, ta, P, st);
        if (P.m <= 8) return launch_tc<FMT, 16, 8, 0, GATED>(tw, ta, P, st);
    }
    return launch_tc<FMT, NTOK, NTOK, 0, GATED>(tw, ta, P, st);
}

bool al(const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; }

} /* anonymous namespace */

bool tc_fp8a8_ok(const R3dGemmQ& p) {
    return p.m >= 1 && p.m <= 64 && (p.k % 128) == 0 && al(p.b, 16) && (p.b_pitch % 16) == 0 &&
           al(p.a, 16) && (p.a_pitch % 16) == 0 && encode_fn() != nullptr;
}
bool tc_mxfp4a8_ok(const R3dGemmQ& p) {
    return p.m >= 1 && p.m <= 32 && (p.k % 128) == 0 && al(p.b, 32) && (p.b_pitch % 32) == 0 &&
           al(p.b_scale, 4) && (p.bs_pitch % 4) == 0 && al(p.a, 16) && (p.a_pitch % 16) == 0 &&
           encode_fn() != nullptr;
}

int tc_fp8a8(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push) {
    const int ntok = p.m <= 16 ? 16 : p.m <= 32 ? 32 : 64;
    const CUtensorMap* tw = tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, kTileRows);
    const CUtensorMap* ta = tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)ntok);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    TcParams P{};
    P.ws = (const uint8_t*)p.b_scale; P.ws_pitch = p.bs_pitch;
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.y = p.y; P.y_pitch = p.y_pitch; P.y_dtype = RAD_BF16;
    P.m = p.m; P.mlive = p.m; P.n = p.n; P.k = p.k;
    P.as_cols = p.as_cols; P.ws_cols = p.bs_cols; P.rblk = p.rblk; P.ws_dtype = p.bs_dtype;
    if (push) P.push = *push;
    if (ntok == 16) return launch_tc_ml<TC_FP8, 16>(tw, ta, P, st);
    if (ntok == 32) return launch_tc_ml<TC_FP8, 32>(tw, ta, P, st);
    return launch_tc_ml<TC_FP8, 64>(tw, ta, P, st);
}

/* gemm_nt_q_gated in one launch: served when the plain band would run the same accumulation (one CTA a
 * row tile over the whole K: enough tiles that K is not split), so that the result stays byte-identical to
 * the band followed by the quantiser; n_half a multiple of 128 = one quantiser group a gate tile */
bool tc_fp8a8_gated_ok(const R3dGemmQ& p) {
    const int tiles = (p.n + kTileRows - 1) / kTileRows;
    return tc_fp8a8_ok(p) && (p.n % (2 * kTileRows)) == 0 && k_shares(tiles, p.k / kStageK, 2) == 1;
}

int tc_fp8a8_gated(const R3dGemmQ& p, const GatedOut& g, cudaStream_t st) {
    const int ntok = p.m <= 16 ? 16 : p.m <= 32 ? 32 : 64;
    const CUtensorMap* tw = tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, kTileRows);
    const CUtensorMap* ta = tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)ntok);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    TcParams P{};
    P.ws = (const uint8_t*)p.b_scale; P.ws_pitch = p.bs_pitch;
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.y = nullptr; P.y_pitch = 0; P.y_dtype = RAD_BF16;
    P.m = p.m; P.mlive = p.m; P.n = p.n; P.k = p.k;
    P.as_cols = p.as_cols; P.ws_cols = p.bs_cols; P.rblk = p.rblk; P.ws_dtype = p.bs_dtype;
    P.gated = 1; P.gsilu = g.silu; P.gob_dtype = g.ob_dtype;
    P.gq = (uint8_t*)g.q; P.gq_pitch = g.q_pitch; P.gs = g.scale; P.gs_pitch = g.s_pitch;
    P.gob = g.ob; P.gob_pitch = g.ob_pitch;
    if (ntok == 16) return launch_tc_ml<TC_FP8, 16, 1>(tw, ta, P, st);
    if (ntok == 32) return launch_tc_ml<TC_FP8, 32, 1>(tw, ta, P, st);
    return launch_tc_ml<TC_FP8, 64, 1>(tw, ta, P, st);
}

int tc_mxfp4a8(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push) {
    const int ntok = p.m <= 16 ? 16 : 32;
    const CUtensorMap* tw = tensor_map(p.b, (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.b_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, kTileRows);
    const CUtensorMap* ta = tensor_map(p.a, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.a_pitch,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)ntok);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    TcParams P{};
    P.ws = (const uint8_t*)p.b_scale; P.ws_pitch = p.bs_pitch;
    P.as = p.a_scale; P.as_pitch = p.as_pitch;
    P.y = p.y; P.y_pitch = p.y_pitch; P.y_dtype = RAD_BF16;
    P.m = p.m; P.mlive = p.m; P.n = p.n; P.k = p.k;
    P.as_cols = p.as_cols; P.ws_cols = p.bs_cols; P.rblk = 1; P.ws_dtype = RAD_E8M0;
    if (push) P.push = *push;
    if (ntok == 16) return launch_tc_ml<TC_MXFP4, 16>(tw, ta, P, st);
    return launch_tc_ml<TC_MXFP4, 32>(tw, ta, P, st);
}

bool tc_logits_ok(const R3dLogits& l) {
    if (l.head_fmt == 1)                      /* mxfp4 head: e2m1 nibbles + one E8M0 byte per 32 columns */
        return l.m >= 1 && l.m <= 16 && l.k >= 128 && (l.k % 128) == 0 && l.k <= kLgMaxK && al(l.codes, 32) &&
               (l.code_pitch % 32) == 0 && al(l.scale, 4) && (l.scale_pitch % 4) == 0 && al(l.x, 8) &&
               (l.x_pitch % 4) == 0 && (l.y_dtype == RAD_F32 || l.y_dtype == RAD_BF16) && encode_fn() != nullptr;
    return l.head_fmt == 0 && l.m >= 1 && l.m <= kLgMaxTok && l.k >= 128 && (l.k % 128) == 0 &&
           l.k <= kLgMaxK && (l.br == 1 || l.br == 128) && al(l.codes, 16) && (l.code_pitch % 16) == 0 &&
           al(l.x, 8) && (l.x_pitch % 4) == 0 &&
           (l.scale_dtype == RAD_BF16 || l.scale_dtype == RAD_F16 || l.scale_dtype == RAD_F32) &&
           (l.y_dtype == RAD_F32 || l.y_dtype == RAD_BF16) && encode_fn() != nullptr;
}

/* Two launches: the activation split (a few microseconds of work on M x K elements), then the
 * weight-streaming kernel with the piece rows as its "tokens". The scratch between them is a
 * file-scope device array: calls must be ordered on one stream (or otherwise serialised). */
int tc_logits(const R3dLogits& l, cudaStream_t st, const PushCfg* push) {
    LgScratch sc;
    if (!lg_scratch(&sc)) return RAD_E_DEVICE;
    const int mp = l.m <= 1 ? 1 : l.m <= 2 ? 2 : l.m <= 4 ? 4 : l.m <= 8 ? 8 : l.m <= 16 ? 16 : 32;
    const int n128 = l.k / 128;
    count_launch();
    {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)((mp * n128 + 3) / 4)); cfg.blockDim = dim3(128); cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = tc_pdl_on() ? 1 : 0;
        if (cudaLaunchKernelEx(&cfg, k_lg_split, (const uint16_t*)l.x, (int64_t)l.x_pitch, (int)l.m, mp, (int)l.k,
                               sc.pieces, sc.scale) != cudaSuccess) return RAD_E_DEVICE;
    }
    const int ntok = 2 * mp <= 16 ? 16 : 2 * mp;
    const bool fp4 = l.head_fmt == 1;
    const CUtensorMap* tw = tensor_map(l.codes, (uint64_t)l.k, (uint64_t)l.n, (uint64_t)l.code_pitch,
                                       fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                                       kTileRows);
    const CUtensorMap* ta = tensor_map(sc.pieces, (uint64_t)l.k, (uint64_t)(2 * mp), (uint64_t)l.k,
                                       CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)ntok);
    if (!tw || !ta) return RAD_E_UNSUPPORTED;
    TcParams P{};
    P.ws = (const uint8_t*)l.scale; P.ws_pitch = l.scale_pitch;
    P.as = sc.scale; P.as_pitch = n128;
    P.y = l.y; P.y_pitch = l.y_pitch; P.y_dtype = l.y_dtype;
    P.m = 2 * mp; P.mlive = l.m; P.n = l.n; P.k = l.k;
    P.as_cols = n128; P.ws_cols = n128; P.rblk = l.br; P.ws_dtype = l.scale_dtype;
    if (push) P.push = *push;
    if (fp4) {
        /* the mxfp4 head: the tensor core applies the E8M0 group scales (one byte per 32 columns),
         * the epilogue only the pieces' power-of-two scales */
        P.ws_cols = l.k / 32; P.rblk = 1; P.ws_dtype = RAD_E8M0;
        switch (mp) {
        case 1:  return launch_tc<TC_MXFP4, 16, 2, 1>(tw, ta, P, st);
        case 2:  return launch_tc<TC_MXFP4, 16, 4, 1>(tw, ta, P, st);
        case 4:  return launch_tc<TC_MXFP4, 16, 8, 1>(tw, ta, P, st);
        case 8:  return launch_tc<TC_MXFP4, 16, 16, 1>(tw, ta, P, st);
        default: return launch_tc<TC_MXFP4, 32, 32, 1>(tw, ta, P, st);
        }
    }
    switch (mp) {
    case 1:  return launch_tc<TC_FP8, 16, 2, 1>(tw, ta, P, st);
    case 2:  return launch_tc<TC_FP8, 16, 4, 1>(tw, ta, P, st);
    case 4:  return launch_tc<TC_FP8, 16, 8, 1>(tw, ta, P, st);
    case 8:  return launch_tc<TC_FP8, 16, 16, 1>(tw, ta, P, st);
    case 16: return launch_tc<TC_FP8, 32, 32, 1>(tw, ta, P, st);
    default: return launch_tc<TC_FP8, 64, 64, 1>(tw, ta, P, st);
    }
}

const CUtensorMap* tc_tensor_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                                 CUtensorMapDataType dt, uint32_t box1, uint32_t box0, int promo128) {
    return tensor_map(ptr, d0, d1, pitch_bytes, dt, box1, box0, promo128);
}
int tc_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kTcMaxDevices) return -1;
    return dev;
}
bool tc_have_encoder() { return encode_fn() != nullptr; }
int tc_sm_count() { return sm_count(); }
bool tc_pdl_on() {
    static const bool off = [] { const char* e = getenv("R3D_NO_PDL"); return e && *e && *e != '0'; }();
    return !off;
}

int tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) return v;
    v = tc_mxf4_status();
    if (v) return v;
    v = tc_q8x_status();
    if (v) return v;
    v = tc_gemm2_status();
    if (v) return v;
    v = tc_w2a8_status();
    if (v) return v;
    v = rerank_status();
    return v ? v : tc_gemm_status();
}

} /* namespace r3d */

/* kern_tc_q8x.cu -- the int8-per-32 activation arm of the mxfp4a8 decode band on the tensor core.
 *
 * Contract (src/r3d_gemm_mxfp4.hip:1143-1166, :1268-1281, :1319-1340 of libr3d), bit for bit:
 *   requant   per (token m, 32-of-K group g): e = dec_e4m3(a); mx = max|e|; s = mx ? mx/127 : 1;
 *             x8 = (int8) rintf(e / s); SG[m,g] = s
 *   dot       p = sum x8 * (2 * e2m1)                       exact int32 over the group
 *             c = ((((float)p * SG[m,g]) * AS[m,g/4]) * 2^(x-127)) * 0.5f
 *   walk 0    per 256-of-K step T = ((c0+c1)+(c2+c3)) + ((c4+c5)+(c6+c7)); acc += T
 *   walk 1    lane (g mod 32) adds its groups in ascending order; the 32 lane sums fold by a
 *             butterfly over lane xor 1, 2, 4, 8, 16 (a balanced tree in lane order)
 *
 * The integer dot is what the tensor core computes here, on the packed nibble plane as it lies in
 * HBM (no repacked int8 plane, no expansion in registers). tcgen05.mma kind::mxf4 multiplies
 * e2m1 by e2m1, so the int8 activation is written as three e2m1 digit rows
 *     |x8| = d0 + 4 d1 + 16 d2,   d0 in 0..3,  d1 in -4..3,  d2 in {0,1,2,3,4,6,8}
 * (a top digit of 5 or 7 is not twice an e2m1 value: it becomes 6 or 8 and the middle digit drops
 * by 4), each digit stored as the e2m1 code of digit/2 with the sign of x8. A K=64 instruction
 * spans two 32-groups, whose dots must stay apart: every digit row exists twice, once with the
 * odd groups zeroed and once with the even groups zeroed ("parity" rows). The weights' and the
 * digits' hardware scale factors are constants: 2^0 for the weights (their E8M0 byte enters the
 * float chain at its own place) and 2^2 for the digits, so an accumulator column holds
 * sum (w8/2) * (digit/2) * 4 = sum w8 * digit exactly (small integers in f32). Two forms:
 *   HW = false  digit rows are separate MMA columns; the epilogue forms p = D0 + 4 D1 + 16 D2
 *               (up to four tokens)
 *   HW = true   three MMAs accumulate into one column with digit scales 2^2, 2^4, 2^6: the
 *               column holds p itself (eight tokens: fewer columns, fewer registers)
 * Both were checked bit for bit against the CPU checker on the full 27648 x 5120 plane, on the
 * largest dots there are (|p| = 32 * 127 * 12) and on every int8 value the requantiser can produce.
 * Every accumulator is fresh per 64 of K (no accumulation across groups), the epilogue thread of
 * a weight row reads its columns from tensor memory one 128-of-K unit ahead of the unit it is
 * computing, and runs the float chain above in the reference's order, two groups per packed
 * f32x2 instruction (each half an IEEE f32 operation). For walk 1 the K stages are visited class by
 * class (stage index mod 4 = lane index / 8), so that only eight lane sums per token are live at
 * a time: class r finishes lanes 8r..8r+7, their subtree ((a0+a1)+(a2+a3))+((a4+a5)+(a6+a7)) is
 * final and the four subtrees fold as (P0+P1)+(P2+P3) -- the butterfly's tree. The class order is
 * rotated per CTA (the subtrees are independent).
 *
 * Data path: weights by TMA (plain byte tensor map, 128-byte row segments, 256 K per stage), all
 * E8M0 bytes of the CTA's 128 rows resident in shared memory (one TMA tile per 1024 K), digit
 * rows by TMA from a file-scope device array a small split kernel fills once per call (it also
 * writes x8 and SG into the caller's scratch, the arm's contract). Warp 0 TMA producer, warp 1 MMA
 * issuer and TMEM owner, warps 2.. epilogue (thread = weight row; at eight tokens two warp sets
 * share the tokens). Programmatic dependent launch: weights and their scales are requested
 * before griddepcontrol.wait, everything the previous kernel may have written after it. Every
 * wait is bounded; on expiry a status word is set and the CTA drains, frees its TMEM and leaves
 * without storing.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#define R3D_TC_STATUS_WORD ::r3d::g_tcq_status
namespace r3d { __device__ int g_tcq_status = 0; }
#include "tc_common.cuh"

namespace r3d {

namespace {
using namespace tcdev;

constexpr int kRows = 128;
constexpr int kStageK = 256;                       /* K elements per stage = 128 packed bytes per row */
constexpr int kWBytes = kRows * 128;               /* 16 KiB of weights per stage */
constexpr int kMaxTok = 8;
constexpr int kMaxK = 32768;
constexpr int kPitch = kMaxK / 2;                  /* digit rows: fixed pitch, so the zeroed halves never move */
constexpr int kDigitRows = 48;
constexpr int kSfCols = 32;                        /* scale-factor words: 8 columns each for weights, digit 0, 1, 2 */
constexpr int kTmemCols = 256;
constexpr int kMaxStages = 8;
constexpr int kScTile = kRows * 32;                /* E8M0 bytes of 128 rows x 1024 K */

/* MT tokens (1, 2, 4, 8; M rounds up), HW digit sum by the tensor core, EW epilogue warp sets (each
 * set = four warps = the 128 weight rows; the sets share the tokens) */
template <int MT, bool HW, int EW>
struct Shape {
    static constexpr int TPS = MT / EW;                                /* tokens per set */
    static constexpr int CPT = HW ? 2 : 6;                             /* columns per token per K=64 slab */
    static constexpr int SB = HW ? TPS * 2 : (TPS == 1 ? 8 : (TPS == 2 ? 16 : 24));   /* columns of one set */
    static constexpr int NP = HW ? 16 : (EW * SB <= 16 ? 16 : (EW * SB <= 32 ? 32 : 48));
    static constexpr int UC = 2 * NP;                                  /* columns of a 128-K unit */
    static constexpr int kBufs = (kTmemCols - kSfCols) / UC > 4 ? 4 : (kTmemCols - kSfCols) / UC;
    static constexpr int kPBytes = (HW ? 48 : NP) * 128;               /* digit tile bytes per stage */
    static constexpr int kStage = kWBytes + kPBytes;
    static constexpr int kThreads = 64 + 128 * EW;
    static_assert(MT % EW == 0 && TPS >= 1 && TPS <= 4 && EW * SB <= 48, "token split");
};

/* digit row of (token t, parity, digit j) inside the 48-row digit plane. In every form the
 * parity is the row's lowest bit: a row is only ever written at groups of its own parity, whatever
 * M the calls of a process bring, so its other half stays zero for good. */
__host__ __device__ inline int digit_row(bool hw, int tps, int sb, int t, int par, int j) {
    return hw ? j * 16 + t * 2 + par : (t / tps) * sb + (t % tps) * 6 + j * 2 + par;
}

/* two f32 in one 64-bit register pair and the packed arithmetic on them (each half is an IEEE
 * round-to-nearest f32 operation, the same bits as the scalar instruction): half the issue slots */
typedef uint64_t f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r;
}

struct PQ {
    const float* as; int64_t as_pitch;
    const float* sg;                                /* f32 [M, K/32], the split kernel's output */
    uint16_t* y; int64_t y_pitch;
    int m, n, k, stages;
};

__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}

/* ring position: slot index and the phase bit of its current lap */
struct Ring {
    int i = 0; uint32_t ph = 0; int n;
    __device__ explicit Ring(int n_) : n(n_) {}
    __device__ void next() { if (++i == n) { i = 0; ph ^= 1u; } }
};

template <int N>
__device__ __forceinline__ void ld_cols(uint32_t ta, float* v) {
    if (N == 24) { tmem_ld16(ta, v); tmem_ld8(ta + 16, v + 16); }
    else tmem_ld<N>(ta, v);
}

template <int MT, int WALK, bool HW, int EW>
__global__ void __launch_bounds__(Shape<MT, HW, EW>::kThreads, 2)
k_tc_q8x(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
         const __grid_constant__ CUtensorMap tmP, const PQ P) {
    using S = Shape<MT, HW, EW>;
    constexpr int TPS = S::TPS, SB = S::SB, NP = S::NP, UC = S::UC, kBufs = S::kBufs;
    static_assert(kSfCols + kBufs * UC <= kTmemCols && kBufs >= 2, "TMEM columns");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int kStages = P.stages;
    const int nk = P.k / kStageK;
    const int n128 = P.k / 128;
    const int ntile = (nk + 3) / 4;
    uint8_t* sc = smem + kStages * S::kStage;                       /* [ntile][128 rows][32 bytes] */
    uint64_t* full = (uint64_t*)(sc + ntile * kScTile);             /* weights of a stage have landed */
    uint64_t* pfull = full + kMaxStages;                            /* digit tile of a stage has landed */
    uint64_t* empty = pfull + kMaxStages;                           /* the stage's MMAs have read it */
    uint64_t* acc_full = empty + kMaxStages;
    uint64_t* acc_empty = acc_full + 4;
    uint64_t* sc_full = acc_empty + 4;
    uint64_t* sf_ready = sc_full + 1;
    uint32_t* tmem_slot = (uint32_t*)(sf_ready + 1);
    float* rec_s = (float*)(tmem_slot + 4);                         /* [MT][n128] records of 8 floats: SG of the
                                                                       unit's four groups, AS twice, two unused */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = blockIdx.x * kRows;
    /* walk 1 visits the four stage classes in a rotated order, a different start per CTA: classes 2c
     * and 2c+1 share 256-byte blocks of a weight row, so a class is either all first touches (DRAM)
     * or all second touches (L2); mixing the phases across CTAs keeps DRAM busy throughout */
    const int rs = WALK ? (int)(blockIdx.x & 3u) : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&pfull[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < kBufs; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4 * EW); }
        mbar_init(sc_full, 1); mbar_init(sf_ready, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    dep_launch();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 1) {
        tc_fence_before();
        asm volatile("bar.sync 2, %0;" ::"n"(S::kThreads - 32) : "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = warp >= 1 ? *tmem_slot : 0u;
    bool alive = true;

    if (warp == 0) {
        /* ---------------- TMA producer ----------------
         * Weights and their scale bytes depend on nothing that runs before this kernel: the scale
         * tiles and the first ring of weights are requested at once. The digit tiles are the split
         * kernel's output and are requested only after dep_wait(). */
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmP) : "memory");
            mbar_expect_tx(sc_full, (uint32_t)(ntile * kScTile));
            for (int tl = 0; tl < ntile; ++tl) tma_load_2d(sc + tl * kScTile, &tmS, tl * 32, r0, sc_full);
            auto digits = [&](int slot, int st) {
                uint8_t* dst = smem + slot * S::kStage + kWBytes;
                mbar_expect_tx(&pfull[slot], (uint32_t)S::kPBytes);
                if (HW) {
#pragma unroll
                    for (int j = 0; j < 3; ++j) tma_load_2d(dst + j * 2048, &tmP, st * 128, j * 16, &pfull[slot]);
                } else {
                    tma_load_2d(dst, &tmP, st * 128, 0, &pfull[slot]);
                }
            };
            const int first = nk < kStages ? nk : kStages;
            int held[kMaxStages];                                  /* stages whose digits wait for dep_wait() */
            int v = 0;
            Ring rg(kStages);
            bool ok = true;
            for (int ri = 0; ri < (WALK ? 4 : 1) && ok; ++ri) {
                for (int st = WALK ? ((rs + ri) & 3) : 0; st < nk; st += (WALK ? 4 : 1)) {
                    if (!mbar_wait(&empty[rg.i], rg.ph ^ 1u, 22)) { ok = false; break; }
                    mbar_expect_tx(&full[rg.i], (uint32_t)kWBytes);
                    tma_load_2d(smem + rg.i * S::kStage, &tmW, st * 128, r0, &full[rg.i]);
                    if (v < first) {
                        held[v] = st;
                        if (v == first - 1) {
                            dep_wait();
                            for (int j = 0; j < first; ++j) digits(j, held[j]);
                        }
                    } else {
                        digits(rg.i, st);
                    }
                    ++v; rg.next();
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (elect_one()) {
            /* instruction descriptor, block-scaled kinds: a/b format e2m1 (1), K-major operands,
             * N >> 3 at bit 17, scale format ue8m0 at bit 23, M >> 4 at bit 24 */
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | (1u << 23) |
                                   ((uint32_t)(kRows >> 4) << 24);
            Ring rg(kStages), ab(kBufs);
            bool ok = mbar_wait(sf_ready, 0, 23);
            for (int ri = 0; ri < (WALK ? 4 : 1) && ok; ++ri) {
                for (int st = WALK ? ((rs + ri) & 3) : 0; st < nk && ok; st += (WALK ? 4 : 1)) {
                    if (!mbar_wait(&full[rg.i], rg.ph, 25) || !mbar_wait(&pfull[rg.i], rg.ph, 29)) { ok = false; break; }
                    const uint32_t a0 = smem_u32(smem + rg.i * S::kStage), b0 = a0 + kWBytes;
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        if (!mbar_wait(&acc_empty[ab.i], ab.ph ^ 1u, 24)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int sl = 0; sl < 2; ++sl) {
                            const int i = 2 * u + sl;
                            const uint32_t d = tmem_base + kSfCols + ab.i * UC + sl * NP;
                            if (HW) {
#pragma unroll
                                for (int j = 0; j < 3; ++j)
                                    umma_mxf4(d, smem_desc_sw128(a0 + i * 32), smem_desc_sw128(b0 + j * 2048 + i * 32),
                                              idesc, tmem_base, tmem_base + 8 + 8 * j, (uint32_t)(j > 0));
                            } else {
                                umma_mxf4(d, smem_desc_sw128(a0 + i * 32), smem_desc_sw128(b0 + i * 32), idesc,
                                          tmem_base, tmem_base + 8, 0u);
                            }
                        }
                        umma_commit(&acc_full[ab.i]);
                        ab.next();
                    }
                    umma_commit(&empty[rg.i]);
                    rg.next();
                }
            }
        }
    } else {
        /* ---------------- epilogue: thread = weight row, warp set = token share ---------------- */
        const int q = warp & 3;                                    /* TMEM lane quarter */
        const int set = (warp - 2) >> 2;
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        if (set == 0) {
            /* constant scale factors: weights 2^0, digits 2^2 (and 2^4, 2^6 in the accumulating form) */
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                tmem_st1(tlane + c, 0x7f7f7f7fu);
                tmem_st1(tlane + 8 + c, 0x81818181u);
                tmem_st1(tlane + 16 + c, 0x83838383u);
                tmem_st1(tlane + 24 + c, 0x85858585u);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sf_ready);
        }
        /* the requantised activation's scales are the previous kernels' output */
        dep_wait();
        const int et = threadIdx.x - 64;
        for (int i = et; i < MT * n128; i += 128 * EW) {
            const int t = i / n128, c = i - t * n128;
            float4 sg4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float as = 0.0f;
            if (t < P.m) {
                sg4 = __ldg((const float4*)(P.sg + (int64_t)t * (4 * n128) + 4 * c));
                as = __ldg(P.as + (int64_t)t * P.as_pitch + c);
            }
            *(float4*)(rec_s + 8 * i) = sg4;
            *(float2*)(rec_s + 8 * i + 4) = make_float2(as, as);
        }
        asm volatile("bar.sync 3, %0;" ::"n"(128 * EW) : "memory");
        alive = mbar_wait(sc_full, 0, 26);

        /* Groups travel in pairs (g, g+1) = the two halves of a 64-bit register pair: adjacent
         * accumulator columns, adjacent SG values, one packed instruction per step of both chains. */
        float acc[TPS], half[TPS], sub[TPS][4];        /* sub: subtree of the ri-th class visited */
        f32x2 la[TPS][4];                                /* walk 1: lane sums (8r+2i, 8r+2i+1) of the current class */
#pragma unroll
        for (int t = 0; t < TPS; ++t) {
            acc[t] = 0.0f; half[t] = 0.0f; sub[t][0] = sub[t][1] = sub[t][2] = sub[t][3] = 0.0f;
#pragma unroll
            for (int l = 0; l < 4; ++l) la[t][l] = 0ull;
        }
        const uint8_t* sc_row = sc + (q * 32 + lane) * 32;
        const uint32_t tset = tlane + kSfCols + set * SB;
        const float* rec_t = rec_s + (size_t)(set * TPS) * n128 * 8;
        const f32x2 k_half = pk2(0.5f, 0.5f), k_four = pk2(4.0f, 4.0f), k_sixteen = pk2(16.0f, 16.0f);
        const float nzf = P.m < 0 ? 1.0f : -0.0f;                   /* -0 the assembler cannot fold away */
        const f32x2 k_nz = pk2(nzf, nzf);
        /* The walk is a sequence of steps of one 128-of-K unit (two K=64 slabs, four 32-groups), two
         * per stage. The tensor-memory loads of step i+1 are issued before step i is computed and
         * waited for after it, so their latency hides behind the float chains. What a step keeps of
         * its loads is the integer dot of every (token, group) as a float, two groups per register
         * pair: PF; the raw columns (three digit columns per dot when the digits are summed here) are
         * live only while the load is in flight. */
        float raw[2][SB];
        f32x2 PF[TPS][2];
        Ring ab(kBufs);                                  /* accumulator unit of the step being fetched */
        auto fetch = [&]() -> bool {
            if (!mbar_wait(&acc_full[ab.i], ab.ph, 28)) return false;
            tc_fence_after();
            ld_cols<SB>(tset + ab.i * UC, raw[0]);
            ld_cols<SB>(tset + ab.i * UC + NP, raw[1]);
            return true;
        };
        auto landed = [&]() {
            tmem_ld_wait();
            tmem_pin<SB>(raw[0]);
            tmem_pin<SB>(raw[1]);
            tc_fence_before();
            __syncwarp();
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.eq.u32 p, %1, 0;\n\t"
                "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
                ::"r"(smem_u32(&acc_empty[ab.i])), "r"((uint32_t)lane) : "memory");
            ab.next();
#pragma unroll
            for (int tl = 0; tl < TPS; ++tl)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float* col = raw[h] + tl * S::CPT;
                    f32x2 pf = pk2(col[0], col[1]);
                    if (!HW) pf = fma2(pk2(col[4], col[5]), k_sixteen, fma2(pk2(col[2], col[3]), k_four, pf));
                    PF[tl][h] = pf;
                }
        };
        constexpr int kStep = WALK ? 4 : 1;
        /* (ri, st): ri-th class visited (class (rs + ri) & 3) and the stage within it; classes
         * without a stage (K < 1024) are skipped: their lanes hold +0 and so does their subtree */
        int ri = 0, st = rs;
        while (WALK && ri < 4 && st >= nk) { ++ri; st = (rs + ri) & 3; }
        if (ri >= 4) alive = false;                      /* cannot happen: nk >= 1 */
        if (alive) { alive = fetch(); if (alive) landed(); }
        while (alive) {
            int nst = st + kStep, nri = ri;
            if (WALK) while (nst >= nk && nri < 4) { ++nri; nst = (rs + nri) & 3; }
            const bool has_next = nst < nk && nri < 4;
            const uint2 sw = *(const uint2*)(sc_row + (st >> 2) * kScTile + (st & 3) * 8);
            /* bytes 0x00 (2^-127, a subnormal) and 0xFF (NaN) are not "byte << 23": rare, so one test per stage */
            const uint32_t any = (((sw.x - 0x01010101u) & ~sw.x) | ((sw.y - 0x01010101u) & ~sw.y) |
                                  ((~sw.x - 0x01010101u) & sw.x) | ((~sw.y - 0x01010101u) & sw.y)) & 0x80808080u;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                bool fetched = false;
                if (u == 0 || has_next) { alive = fetch(); fetched = alive; }
                if (!alive) break;
                const uint32_t word = u ? sw.y : sw.x;
                f32x2 sc01, sc23;
                if (any) {
                    sc01 = pk2(e8m0_to_f32((uint8_t)word), e8m0_to_f32((uint8_t)(word >> 8)));
                    sc23 = pk2(e8m0_to_f32((uint8_t)(word >> 16)), e8m0_to_f32((uint8_t)(word >> 24)));
                } else {
                    sc01 = pk2(__uint_as_float((word << 23) & 0x7f800000u), __uint_as_float((word << 15) & 0x7f800000u));
                    sc23 = pk2(__uint_as_float((word << 7) & 0x7f800000u), __uint_as_float((word >> 1) & 0x7f800000u));
                }
                const float* rec_u = rec_t + (2 * st + u) * 8;
#pragma unroll
                for (int tl = 0; tl < TPS; ++tl) {
                    const float* rec = rec_u + (size_t)tl * n128 * 8;
                    const ulonglong2 sg = *(const ulonglong2*)rec;          /* (SG0, SG1), (SG2, SG3) */
                    const f32x2 as2 = *(const f32x2*)(rec + 4);              /* (AS, AS) */
                    f32x2 c[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {                            /* slab h: groups 2h, 2h+1 */
                        f32x2 v = mul2(PF[tl][h], h ? sg.y : sg.x);
                        v = mul2(v, as2);
                        v = mul2(v, h ? sc23 : sc01);
                        /* walk 1 adds the pair with a packed add: the halving is written as fma(v, 0.5, -0) so
                         * that it is rounded alone (a packed multiply whose only use is a packed add is merged
                         * into one fused multiply-add by the assembler; with a subnormal half that is another
                         * rounding than the chain's) */
                        c[h] = WALK ? fma2(v, k_half, k_nz) : mul2(v, k_half);
                    }
                    if (WALK == 0) {
                        float c0, c1, c2, c3;
                        upk2(c[0], c0, c1); upk2(c[1], c2, c3);
                        const float hsum = __fadd_rn(__fadd_rn(c0, c1), __fadd_rn(c2, c3));
                        if (u == 0) half[tl] = hsum;
                        else acc[tl] = __fadd_rn(acc[tl], __fadd_rn(half[tl], hsum));
                    } else {
                        la[tl][2 * u] = add2(la[tl][2 * u], c[0]);
                        la[tl][2 * u + 1] = add2(la[tl][2 * u + 1], c[1]);
                    }
                }
                if (fetched) landed();
            }
            if (!alive) break;
            if (WALK && (!has_next || nri != ri)) {
                /* the class is complete: its eight lanes of the butterfly fold to their subtree */
#pragma unroll
                for (int t = 0; t < TPS; ++t) {
                    float a[8];
#pragma unroll
                    for (int l = 0; l < 4; ++l) { upk2(la[t][l], a[2 * l], a[2 * l + 1]); la[t][l] = 0ull; }
                    const float p = __fadd_rn(__fadd_rn(__fadd_rn(a[0], a[1]), __fadd_rn(a[2], a[3])),
                                              __fadd_rn(__fadd_rn(a[4], a[5]), __fadd_rn(a[6], a[7])));
#pragma unroll
                    for (int c = 0; c < 4; ++c) if (ri == c) sub[t][c] = p;
                }
            }
            if (!has_next) break;
            st = nst; ri = nri;
        }
        const int row = r0 + q * 32 + lane;
        if (alive && row < P.n) {
#pragma unroll
            for (int tl = 0; tl < TPS; ++tl) {
                const int t = set * TPS + tl;
                if (t >= P.m) break;
                float v = acc[tl];
                if (WALK) {
                    /* class c was visited as number (c - rs) & 3: (P0 + P1) + (P2 + P3) */
                    const float* s4 = sub[tl];
                    v = rs == 0 ? __fadd_rn(__fadd_rn(s4[0], s4[1]), __fadd_rn(s4[2], s4[3]))
                      : rs == 1 ? __fadd_rn(__fadd_rn(s4[3], s4[0]), __fadd_rn(s4[1], s4[2]))
                      : rs == 2 ? __fadd_rn(__fadd_rn(s4[2], s4[3]), __fadd_rn(s4[0], s4[1]))
                                : __fadd_rn(__fadd_rn(s4[1], s4[2]), __fadd_rn(s4[3], s4[0]));
                }
                P.y[(int64_t)t * P.y_pitch + row] = f32_to_bf16(v);
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

/* ------------------------------------------------------------------ activation split */
__device__ __align__(256) uint8_t g_q8x_digits[kDigitRows * kPitch];

/* One warp per (token, 32-of-K group), lane = element: the arm's requantisation (x8 and SG go to
 * the caller's scratch as the contract says) and the three e2m1 digit codes of x8, packed two per
 * byte (low nibble = even k) into the digit rows of the group's parity. The rows of the other
 * parity are never written at this group's offset: they stay zero from the array's
 * initialisation, because the row pitch is fixed. */
__global__ void __launch_bounds__(256)
k_q8x_split(const uint8_t* __restrict__ a, int64_t a_pitch, int m, int k,
            int8_t* __restrict__ x8o, float* __restrict__ sgo, uint8_t* __restrict__ digits,
            int hw, int tps, int sb) {
    dep_launch();
    dep_wait();                    /* the activation is the previous kernel's output, and the
                                      previous reader of the digit rows must have finished */
    const int cols = k >> 5;
    const int gw = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (gw >= m * cols) return;
    const int t = gw / cols, g = gw - t * cols;
    const int lane = threadIdx.x & 31;
    const float e = e4m3_to_f32(a[(int64_t)t * a_pitch + (g << 5) + lane]);
    float mx = fabsf(e);
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float s = mx ? __fdiv_rn(mx, 127.0f) : 1.0f;
    if (lane == 0) sgo[(int64_t)t * cols + g] = s;
    const int8_t x = (int8_t)rintf(__fdiv_rn(e, s));
    x8o[(int64_t)t * k + (g << 5) + lane] = x;

    const uint32_t ax = (uint32_t)(x < 0 ? -(int)x : (int)x), neg = x < 0 ? 8u : 0u;
    uint32_t h = ax >> 4, l1 = (ax >> 2) & 3u;
    const uint32_t l0 = ax & 3u;
    uint32_t n1;                                               /* middle digit's nibble */
    if (h == 5u || h == 7u) { h += 1u; n1 = (4u - l1) | (neg ^ 8u); }     /* digit l1 - 4: magnitude 1..4 */
    else n1 = l1 ? (l1 | neg) : 0u;
    const uint32_t n0 = l0 ? (l0 | neg) : 0u;
    const uint32_t hc = h <= 4u ? h : (h == 6u ? 5u : 6u);     /* e2m1 code of h/2: 0,.5,1,1.5,2,3,4 */
    const uint32_t n2 = hc ? (hc | neg) : 0u;
    const uint32_t mine = n0 | (n1 << 4) | (n2 << 8);
    /* lane L < 12 writes word w = L % 4 (elements 8w..8w+7) of digit j = L / 4 */
    const int j = lane >> 2, w = lane & 3;
    uint32_t word = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t v = __shfl_sync(0xffffffffu, mine, 8 * w + i);
        word |= ((v >> (4 * (j < 3 ? j : 0))) & 0xfu) << (4 * i);
    }
    if (lane < 12) {
        const int row = digit_row(hw != 0, tps, sb, t, g & 1, j);
        *(uint32_t*)(digits + (int64_t)row * kPitch + g * 16 + w * 4) = word;
    }
}

uint8_t* digit_plane() {
    static uint8_t* per_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!per_dev[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_q8x_digits) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        per_dev[dev] = (uint8_t*)p;
    }
    return per_dev[dev];
}

template <int MT, bool HW, int EW>
size_t smem_bytes(int k, int stages) {
    const int nk = k / kStageK;
    return 1024 + (size_t)stages * Shape<MT, HW, EW>::kStage + (size_t)((nk + 3) / 4) * kScTile +
           (3 * kMaxStages + 10) * sizeof(uint64_t) + 16 + (size_t)MT * (k / 128) * 8 * sizeof(float);
}

/* the deepest ring (3..6 stages) that lets two CTAs share an SM, else the deepest that fits one */
template <int MT, bool HW, int EW>
int pick_stages(int k) {
    const size_t half = 233472 / 2 - 1024, whole = 227 * 1024;
    for (int s = 6; s >= 3; --s) if (smem_bytes<MT, HW, EW>(k, s) <= half) return s;
    for (int s = 6; s >= 3; --s) if (smem_bytes<MT, HW, EW>(k, s) <= whole) return s;
    return 0;
}

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

template <int MT, int WALK, bool HW, int EW>
int run(const R3dGemmQ& p, int8_t* x8, float* sg, cudaStream_t st) {
    using S = Shape<MT, HW, EW>;
    uint8_t* plane = digit_plane();
    if (!plane) return RAD_E_DEVICE;
    const int stages = pick_stages<MT, HW, EW>(p.k);
    if (!stages) return RAD_E_UNSUPPORTED;
    const size_t smem = smem_bytes<MT, HW, EW>(p.k, stages);
    static size_t attr_set[kTcMaxDevices] = {};
    const int dev = tc_device();
    if (dev < 0) return RAD_E_DEVICE;
    if (smem > attr_set[dev]) {
        if (cudaFuncSetAttribute(k_tc_q8x<MT, WALK, HW, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return RAD_E_DEVICE;
        (void)cudaFuncSetAttribute(k_tc_q8x<MT, WALK, HW, EW>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   (int)cudaSharedmemCarveoutMaxShared);
        attr_set[dev] = smem;
    }
    /* walk 1 touches the two 128-byte halves of a 256-byte block of a weight row a quarter of the kernel
     * apart: its weight map promotes L2 fills to 128 bytes, not 256 (measured: 17.6 -> 16.5 us at M = 1) */
    const CUtensorMap* tw = tc_tensor_map(p.b, (uint64_t)(p.k / 2), (uint64_t)p.n, (uint64_t)p.b_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows, 128u, WALK ? 1 : 0);
    const CUtensorMap* ts = tc_tensor_map(p.b_scale, (uint64_t)(p.k / 32), (uint64_t)p.n, (uint64_t)p.bs_pitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, kRows, 32u);
    const CUtensorMap* tp = tc_tensor_map(plane, (uint64_t)(p.k / 2), (uint64_t)kDigitRows, (uint64_t)kPitch,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint32_t)(HW ? 16 : S::NP));
    if (!tw || !ts || !tp) return RAD_E_UNSUPPORTED;

    count_launch();
    const unsigned sgrid = (unsigned)(((int64_t)p.m * (p.k >> 5) + 7) / 8);
    if (launch_pdl(k_q8x_split, dim3(sgrid), dim3(256), 0, st, (const uint8_t*)p.a, (int64_t)p.a_pitch,
                   (int)p.m, (int)p.k, x8, sg, plane, (int)HW, (int)S::TPS, (int)S::SB) != cudaSuccess) return RAD_E_DEVICE;
    PQ P{};
    P.as = p.a_scale; P.as_pitch = p.as_pitch; P.sg = sg;
    P.y = (uint16_t*)p.y; P.y_pitch = p.y_pitch;
    P.m = p.m; P.n = p.n; P.k = p.k; P.stages = stages;
    const int tiles = (p.n + kRows - 1) / kRows;
    count_launch();
    const cudaError_t e = launch_pdl(k_tc_q8x<MT, WALK, HW, EW>, dim3((unsigned)tiles), dim3(S::kThreads), smem, st,
                                     *tw, *ts, *tp, P);
    return e == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

bool al(const void* p, int a) { return (((uintptr_t)p) & (uintptr_t)(a - 1)) == 0; }

} /* anonymous namespace */

bool tc_q8x_ok(const R3dGemmQ& p) {
    static const bool off = [] { const char* e = getenv("R3D_Q8X_NO_TC"); return e && *e && *e != '0'; }();
    if (off) return false;
    if (!(p.m >= 1 && p.m <= kMaxTok && p.k >= 256 && (p.k % 256) == 0 && p.k <= kMaxK && p.as_cols == p.k / 128 &&
          al(p.b, 16) && (p.b_pitch % 16) == 0 && al(p.b_scale, 16) && (p.bs_pitch % 16) == 0 &&
          p.bs_cols == p.k / 32 && tc_have_encoder())) return false;
    return pick_stages<8, true, 2>(p.k) != 0 && pick_stages<4, false, 1>(p.k) != 0;
}

/* Two launches: the split (requantisation + digit rows; the digit plane is a file-scope device
 * array, so calls on one device must be ordered on one stream), then the weight-streaming kernel.
 * Forms (measured on 27648 x 5120): up to four tokens the epilogue sums the digit columns itself and
 * one warp set serves all tokens (two sets, or the tensor core summing the digits with three times
 * the MMAs, were 1 to 6 us slower); eight tokens need the tensor core's sum to fit the registers. */
int tc_q8x(const R3dGemmQ& p, int8_t* x8, float* sg, int walk, cudaStream_t st) {
    if (p.m == 1) return walk ? run<1, 1, false, 1>(p, x8, sg, st) : run<1, 0, false, 1>(p, x8, sg, st);
    if (p.m == 2) return walk ? run<2, 1, false, 1>(p, x8, sg, st) : run<2, 0, false, 1>(p, x8, sg, st);
    if (p.m <= 4) return walk ? run<4, 1, false, 1>(p, x8, sg, st) : run<4, 0, false, 1>(p, x8, sg, st);
    return walk ? run<8, 1, true, 2>(p, x8, sg, st) : run<8, 0, true, 2>(p, x8, sg, st);
}

int tc_q8x_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcq_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

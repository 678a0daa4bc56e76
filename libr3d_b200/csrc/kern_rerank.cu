/* kern_rerank.cu -- logit_rerank over the joined e4m3 LM head: R candidate ids a row rescored
 * exactly and re-sorted.
 *
 * Contract (src/r3d_logit_rerank_e4m3.hip:22-39, :146-206 of libr3d), bit for bit: for row m and
 * candidate r with global id g (local = g - vocab_off; g < 0 or local outside [0, n_vocab) is a pad:
 * id -1, value -inf)
 *     acc (double) = 0; for k ascending: hv = f32(code[local][k]) * scale[local / br][k / 128]  (ONE f32
 *     rounding); acc += (double) f32(x[m][k]) * (double) hv   (the product of two floats is exact
 *     in double, the add rounds); score = (float) acc
 * then R rounds of selection under (larger value; ties to the LOWER id; pads last), ids / values /
 * the optional (id bits, value) pairs plane written in that order.
 *
 * The double chain is serial by definition, so the work is laid out for its latency, not for a
 * tensor core. Two kernels:
 *   k_logit_rerank_chain (whole 128-K blocks, 16-byte aligned head rows, K up to about 12,000): one
 *     warp carries all the row's chains, lane = candidate, one FP64 add instruction for up to 32
 *     chains; sixteen producer warps form the exact products ahead of it in shared memory (see the
 *     kernel's own comment).
 *   k_logit_rerank_e4m3 (everything else): one block of eight warps per row; every warp serves four
 *     candidates at once, eight lanes each: per 128-K block a lane fetches sixteen consecutive codes
 *     of its candidate's head row, forms the sixteen exact products, and the segment's accumulator
 *     takes the 128 products of the block in ascending k through width-8 shuffles -- the same adds
 *     in the same order, four chains per FP64 instruction. Ragged K, unaligned heads and rows too
 *     wide for shared memory take 32-K steps of four codes a lane.
 * The selection runs in one warp over shared memory.
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"
#include <cmath>
#include <cstdlib>

namespace r3d { __device__ int g_rr_status = 0; }
#define R3D_TC_STATUS_WORD ::r3d::g_rr_status
#include "tc_common.cuh"

namespace r3d {

namespace {
constexpr int kMaxR = 32;
constexpr int kWarps = 8;

/* the same in two halves, so that a load issued ahead is not waited for before its value is needed */
__device__ __forceinline__ uint32_t ld_scale_raw(const void* base, int64_t idx, int dt) {
    return dt == RAD_F32 ? ((const uint32_t*)base)[idx] : (uint32_t)((const uint16_t*)base)[idx];
}
__device__ __forceinline__ float scale_of_raw(uint32_t raw, int dt) {
    if (dt == RAD_F32) return __uint_as_float(raw);
    if (dt == RAD_F16) return f16_to_f32((uint16_t)raw);
    return bf16_to_f32((uint16_t)raw);
}

__device__ __forceinline__ float ld_scale_any(const void* base, int64_t idx, int dt) {
    if (dt == RAD_F32) return ((const float*)base)[idx];
    if (dt == RAD_F16) return f16_to_f32(((const uint16_t*)base)[idx]);
    return bf16_to_f32(((const uint16_t*)base)[idx]);
}

/* The R rounds of selection, run by one whole warp over the candidates' ids and scores in shared
 * memory. Without NaN scores the selection's order is a total order (value descending, lower id first,
 * earlier slot first; pads last), so a candidate's place is the count of candidates ahead of it; with a
 * NaN score lane 0 plays the rounds one after the other, as the reference does. */
__device__ __forceinline__ void rerank_select(const int lane, const int32_t* sid, const float* ssc, const int R,
                                              const int64_t m, int32_t* __restrict__ idx, const int64_t idx_rs,
                                              float* __restrict__ val, const int64_t val_rs, float* __restrict__ pairs) {
    const bool mine = lane < R && sid[lane] >= 0;
    const float sv = lane < R ? ssc[lane] : 0.0f;
    const unsigned any_nan = __ballot_sync(0xffffffffu, mine && sv != sv);
    const unsigned livem = __ballot_sync(0xffffffffu, mine);
    if (any_nan == 0u) {
        if (mine) {
            int ahead = 0;
            const int32_t id = sid[lane];
            for (int c = 0; c < R; ++c) {
                if (!((livem >> c) & 1u) || c == lane) continue;
                const float so = ssc[c];
                const int32_t io = sid[c];
                ahead += (so > sv || (so == sv && (io < id || (io == id && c < lane)))) ? 1 : 0;
            }
            idx[m * idx_rs + ahead] = id;
            val[m * val_rs + ahead] = sv;
            if (pairs) { float* p = pairs + (m * R + ahead) * 2; p[0] = __int_as_float(id); p[1] = sv; }
        }
        const int nl = __popc(livem);
        if (lane < R && lane >= nl) {
            idx[m * idx_rs + lane] = -1;
            val[m * val_rs + lane] = -INFINITY;
            if (pairs) { float* p = pairs + (m * R + lane) * 2; p[0] = __int_as_float(-1); p[1] = -INFINITY; }
        }
        return;
    }
    if (lane != 0) return;
    uint32_t used = 0u;
    for (int o = 0; o < R; ++o) {
        int best = -1;
        for (int c = 0; c < R; ++c) {
            if (((used >> c) & 1u) || sid[c] < 0) continue;
            if (best < 0 || ssc[c] > ssc[best] || (ssc[c] == ssc[best] && sid[c] < sid[best])) best = c;
        }
        const int32_t oid = best >= 0 ? sid[best] : -1;
        const float ov = best >= 0 ? ssc[best] : -INFINITY;
        if (best >= 0) used |= 1u << best;
        idx[m * idx_rs + o] = oid;
        val[m * val_rs + o] = ov;
        if (pairs) {
            float* p = pairs + (m * R + o) * 2;
            p[0] = __int_as_float(oid);
            p[1] = ov;
        }
    }
}

__global__ void __launch_bounds__(32 * kWarps)
k_logit_rerank_e4m3(const uint8_t* __restrict__ x, int xdt, int64_t x_rs,
                    const uint8_t* __restrict__ codes, int64_t code_rs,
                    const void* __restrict__ scale, int64_t scale_rs, int br, int sdt,
                    const int32_t* __restrict__ in, int64_t in_rs,
                    int32_t* __restrict__ idx, int64_t idx_rs, float* __restrict__ val, int64_t val_rs,
                    float* __restrict__ pairs, int R, int K, int64_t NV, int64_t voff, int mode) {
    /* mode 0: nothing staged; 1: the activation row in shared memory; 2: also the candidates' head rows and
     * their scales, fetched by one bulk copy a candidate */
    extern __shared__ __align__(16) float xs[];           /* [K] | then [32][K] bytes of head rows, [32][K/128] scales, a barrier */
    const int x_in_smem = mode >= 1;
    __shared__ int32_t sid[kMaxR];
    __shared__ float ssc[kMaxR];
    const int64_t m = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    static_assert(kWarps * 4 >= kMaxR, "one pass over the candidates");
    if (mode == 2 && threadIdx.x == 0) {
        uint64_t* bar0 = (uint64_t*)((float*)((uint8_t*)(xs + K) + (size_t)kMaxR * K) + kMaxR * (K >> 7));
        tcdev::mbar_init(bar0, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (x_in_smem) {
        for (int k = threadIdx.x; k < K; k += blockDim.x)
            xs[k] = xdt == RAD_F32 ? ((const float*)x)[m * x_rs + k] : bf16_to_f32(((const uint16_t*)x)[m * x_rs + k]);
        __syncthreads();
    }
    {
        const int r = warp * 4 + (lane >> 3), j = lane & 7;      /* candidate slot of this 8-lane segment */
        const int64_t g = r < R ? (int64_t)in[m * in_rs + r] : -1;
        const int64_t local = g - voff;
        const bool pad = r >= R || g < 0 || local < 0 || local >= NV;
        const uint8_t* crow = codes + (pad ? 0 : local) * code_rs;
        const int64_t sbase = pad ? 0 : (local / br) * scale_rs;
        const bool al4 = ((((uintptr_t)codes) | (uintptr_t)code_rs) & 3) == 0;
        double acc = 0.0;
        int k0 = 0;
        const bool al16 = ((((uintptr_t)codes) | (uintptr_t)code_rs) & 15) == 0;
        if (mode == 2) {
            /* the candidates' rows arrive by bulk copies (all of the block's in flight at once: one DRAM round
             * trip a call instead of one a 128-K block), the chain then runs out of shared memory */
            const int nblk = K >> 7;
            uint8_t* rows_s = (uint8_t*)(xs + K);
            float* sc_s = (float*)(rows_s + (size_t)kMaxR * K);
            uint64_t* bar = (uint64_t*)(sc_s + kMaxR * nblk);
            if (warp == 0) {
                /* lane = candidate slot of the whole block here */
                const int64_t g0 = lane < R ? (int64_t)in[m * in_rs + lane] : -1;
                const int64_t l0 = g0 - voff;
                const bool live = lane < R && g0 >= 0 && l0 >= 0 && l0 < NV;
                if (live)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(tcdev::smem_u32(rows_s + (size_t)lane * K)), "l"(codes + l0 * code_rs), "r"((uint32_t)K),
                                   "r"(tcdev::smem_u32(bar)) : "memory");
                const unsigned nlive = __popc(__ballot_sync(0xffffffffu, live));
                if (lane == 0) tcdev::mbar_expect_tx(bar, nlive * (uint32_t)K);
            }
            if (!pad)
                for (int b = j; b < nblk; b += 8) sc_s[r * nblk + b] = ld_scale_any(scale, sbase + b, sdt);
            __syncwarp();
            const bool landed = tcdev::mbar_wait(bar, 0, 51);
            if (landed && !pad) {
                const uint8_t* rs = rows_s + (size_t)r * K + 16 * j;
                const unsigned seg = 0xffu << (lane & 24);
                for (int b = 0; b < nblk; ++b) {
                    const uint4 c = *(const uint4*)(rs + (b << 7));
                    const float s = sc_s[r * nblk + b];
                    const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
                    const float* xb = xs + (b << 7) + 16 * j;
                    double p[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float hv = __fmul_rn(e4m3_to_f32((uint8_t)(cw[i >> 2] >> (8 * (i & 3)))), s);
                        p[i] = __dmul_rn((double)xb[i], (double)hv);
                    }
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj)
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            acc = __dadd_rn(acc, __shfl_sync(seg, p[i], jj, 8));
                }
            }
            if (!landed) acc = __longlong_as_double(0x7ff8000000000000ll);   /* the wait ran out: NaN, status word set */
            k0 = K;
        } else if (x_in_smem && al16) {
            /* whole 128-K blocks: a lane holds sixteen consecutive codes of its candidate (one 16-byte
             * load; the segment reads one 128-byte line), the loads of the next two blocks are in flight
             * while this block's 128 products are added -- in ascending k, as above */
            const int nblk = K >> 7;
            uint4 c1 = make_uint4(0, 0, 0, 0), c2 = c1;
            float s1 = 0.f, s2 = 0.f;
            if (!pad && nblk > 0) { c1 = *(const uint4*)(crow + 16 * j); s1 = ld_scale_any(scale, sbase, sdt); }
            if (!pad && nblk > 1) { c2 = *(const uint4*)(crow + 128 + 16 * j); s2 = ld_scale_any(scale, sbase + 1, sdt); }
            for (int b = 0; b < nblk; ++b) {
                const uint4 c = c1;
                const float s = s1;
                c1 = c2; s1 = s2;
                if (!pad && b + 2 < nblk) {
                    c2 = *(const uint4*)(crow + (int64_t)(b + 2) * 128 + 16 * j);
                    s2 = ld_scale_any(scale, sbase + b + 2, sdt);
                }
                const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
                const float* xb = xs + (b << 7) + 16 * j;
                double p[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float hv = __fmul_rn(e4m3_to_f32((uint8_t)(cw[i >> 2] >> (8 * (i & 3)))), s);
                    p[i] = pad ? 0.0 : __dmul_rn((double)xb[i], (double)hv);
                }
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        acc = __dadd_rn(acc, __shfl_sync(0xffffffffu, p[i], jj, 8));
            }
            k0 = nblk << 7;
        }
        for (; k0 < K; k0 += 32) {
            const int k = k0 + 4 * j;
            double p[4] = {0.0, 0.0, 0.0, 0.0};
            if (!pad && k < K) {
                uint32_t cw;
                if (al4 && k + 4 <= K) cw = *(const uint32_t*)(crow + k);
                else {
                    cw = 0u;
                    for (int i = 0; i < 4; ++i) if (k + i < K) cw |= (uint32_t)crow[k + i] << (8 * i);
                }
                const float s = ld_scale_any(scale, sbase + (k >> 7), sdt);      /* k % 4 == 0: one block for all four */
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (k + i >= K) break;
                    const float hv = __fmul_rn(e4m3_to_f32((uint8_t)(cw >> (8 * i))), s);
                    const float xv = x_in_smem ? xs[k + i]
                                               : (xdt == RAD_F32 ? ((const float*)x)[m * x_rs + k + i]
                                                                 : bf16_to_f32(((const uint16_t*)x)[m * x_rs + k + i]));
                    p[i] = __dmul_rn((double)xv, (double)hv);
                }
            }
            const int n = min(32, K - k0);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const double pj = __shfl_sync(0xffffffffu, p[i], jj, 8);
                    if (jj * 4 + i < n) acc = __dadd_rn(acc, pj);
                }
        }
        if (j == 0 && r < R) {
            sid[r] = pad ? -1 : (int32_t)g;
            ssc[r] = pad ? -INFINITY : (float)acc;
        }
    }
    __syncthreads();
    if (warp == 0) rerank_select(lane, sid, ssc, R, m, idx, idx_rs, val, val_rs, pairs);
}
/* two e4m3 codes -> two f32 by the conversion instruction (e4m3 -> f16 is exact for every code, zeros
 * keep their sign, S.1111.111 becomes a NaN), then f16 -> f32 */
__device__ __forceinline__ void e4m3x2_to_f32(uint16_t two, float& lo, float& hi) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(two));
    asm("cvt.f32.f16 %0, %1;" : "=f"(lo) : "h"((uint16_t)(h2 & 0xffffu)));
    asm("cvt.f32.f16 %0, %1;" : "=f"(hi) : "h"((uint16_t)(h2 >> 16)));
}

/* ---- the chain form: whole 128-K blocks, 16-byte aligned head rows.
 * Warp 0 carries all the row's chains at once, lane = candidate: one FP64 add instruction advances
 * up to 32 chains, fed from shared memory, so a row costs K dependent adds (8 cycles each) and no
 * shuffle sits in the chain. Sixteen producer warps form the exact products up to four 128-K chunks
 * ahead, lane = candidate again: four warps a chunk, each a 32-column quarter of it (one whole
 * 32-byte sector of the candidate's head row per lane; 8-byte pieces of a sector per warp measured
 * twice as slow: nine tenths of the issue stalls were waits for those loads), written as
 * [k][candidate] doubles, which both sides touch without bank conflicts. A ring of four chunk
 * buffers with a full and an empty barrier each couples the two sides; every wait is bounded. */
constexpr int kChainWarps = 17;
constexpr int kChunkK = 128;
constexpr int kChainBufs = 4;
constexpr int kChunkDoubles = kChunkK * kMaxR;

__global__ void __launch_bounds__(32 * kChainWarps)
k_logit_rerank_chain(const uint8_t* __restrict__ x, int xdt, int64_t x_rs,
                     const uint8_t* __restrict__ codes, int64_t code_rs,
                     const void* __restrict__ scale, int64_t scale_rs, int br, int sdt,
                     const int32_t* __restrict__ in, int64_t in_rs,
                     int32_t* __restrict__ idx, int64_t idx_rs, float* __restrict__ val, int64_t val_rs,
                     float* __restrict__ pairs, int R, int K, int64_t NV, int64_t voff) {
    extern __shared__ __align__(16) uint8_t chain_smem[];
    double* p_s = (double*)chain_smem;                               /* [kChainBufs][128][32] */
    double* xs = p_s + kChainBufs * kChunkDoubles;                   /* [K], the activation row widened once */
    uint64_t* full = (uint64_t*)(xs + K);
    uint64_t* empty = full + kChainBufs;
    __shared__ int32_t sid[kMaxR];
    __shared__ float ssc[kMaxR];
    const int64_t m = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int b = 0; b < kChainBufs; ++b) { tcdev::mbar_init(&full[b], 4); tcdev::mbar_init(&empty[b], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x)
        xs[k] = (double)(xdt == RAD_F32 ? ((const float*)x)[m * x_rs + k] : bf16_to_f32(((const uint16_t*)x)[m * x_rs + k]));
    __syncthreads();
    const int64_t g = lane < R ? (int64_t)in[m * in_rs + lane] : -1;
    const int64_t local = g - voff;
    const bool pad = lane >= R || g < 0 || local < 0 || local >= NV;
    const int nchunk = K >> 7;
    if (warp == 0) {
        double acc = 0.0;
        /* sixteen products are fetched while the sixteen before them are added, across chunk borders
         * too: the wait for the next chunk and the fetch of its first sixteen sit before the last
         * sixteen adds of this one. The empty asm statements keep the compiler from sinking a fetch
         * down to its add, which would put the shared-memory latency into the chain. */
        double v[16], u[16];
        bool alive = nchunk > 0 ? __all_sync(0xffffffffu, tcdev::mbar_wait(&full[0], 0u, 52)) : true;
        if (alive && nchunk > 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = p_s[i * kMaxR + lane];
        }
        for (int c = 0; c < nchunk && alive; ++c) {
            const int buf = c % kChainBufs;
            const double* pb = p_s + buf * kChunkDoubles + lane;
#pragma unroll 1
            for (int k0 = 0; k0 < kChunkK - 32; k0 += 32) {
#pragma unroll
                for (int i = 0; i < 16; ++i) u[i] = pb[(k0 + 16 + i) * kMaxR];
                asm volatile("" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) acc = __dadd_rn(acc, v[i]);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = pb[(k0 + 32 + i) * kMaxR];
                asm volatile("" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) acc = __dadd_rn(acc, u[i]);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) u[i] = pb[(kChunkK - 16 + i) * kMaxR];
            asm volatile("" ::: "memory");
#pragma unroll
            for (int i = 0; i < 16; ++i) acc = __dadd_rn(acc, v[i]);
            if (c + 1 < nchunk) {
                const int nb = (c + 1) % kChainBufs;
                /* the warp leaves the loop as one: a lane that gave up takes the others with it */
                alive = __all_sync(0xffffffffu, tcdev::mbar_wait(&full[nb], (uint32_t)(((c + 1) / kChainBufs) & 1), 52));
                if (alive) {
                    const double* pn = p_s + nb * kChunkDoubles + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = pn[i * kMaxR];
                }
            }
            asm volatile("" ::: "memory");
#pragma unroll
            for (int i = 0; i < 16; ++i) acc = __dadd_rn(acc, u[i]);
            __syncwarp();
            if (lane == 0) tcdev::mbar_arrive(&empty[buf]);
        }
        if (!alive) acc = __longlong_as_double(0x7ff8000000000000ll);     /* a wait ran out: NaN, status word set */
        if (lane < R) {
            sid[lane] = pad ? -1 : (int32_t)g;
            ssc[lane] = pad ? -INFINITY : (float)acc;
        }
        __syncwarp();
        rerank_select(lane, sid, ssc, R, m, idx, idx_rs, val, val_rs, pairs);
    } else {
        /* producer warp w serves the chunks c = grp, grp + 4, ... (grp = w / 4: always ring buffer grp) and
         * in them the columns [32 sec, 32 sec + 32) (sec = w % 4): a lane reads one whole 32-byte sector of
         * its candidate's head row per chunk, so no fetched byte is dropped. The codes and the scale of its
         * next chunk but one are already in registers; the loop is unrolled by two so that a slot is
         * refilled in place (a register move would wait for the load). */
        const int w = warp - 1, grp = w >> 2, sec = w & 3;
        const uint8_t* crow = codes + (pad ? 0 : local) * code_rs + 32 * sec;
        const int64_t sbase = pad ? 0 : (local / br) * scale_rs;
        constexpr int kAhead = 2;
        uint4 ca[kAhead], cb2[kAhead];
        uint32_t sq[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int c = grp + kChainBufs * u;
            ca[u] = make_uint4(0u, 0u, 0u, 0u); cb2[u] = ca[u]; sq[u] = 0u;
            if (c < nchunk) {
                ca[u] = *(const uint4*)(crow + (int64_t)c * kChunkK);
                cb2[u] = *(const uint4*)(crow + (int64_t)c * kChunkK + 16);
                sq[u] = ld_scale_raw(scale, sbase + c, sdt);
            }
        }
        bool alive = true;
        double* pb = p_s + grp * kChunkDoubles + (32 * sec) * kMaxR + lane;
        for (int j0 = 0; alive; j0 += kAhead) {
            if (grp + kChainBufs * j0 >= nchunk) break;
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int j = j0 + u, c = grp + kChainBufs * j;
                if (c >= nchunk || !alive) break;
                if (j >= 1) alive = __all_sync(0xffffffffu, tcdev::mbar_wait(&empty[grp], (uint32_t)((j - 1) & 1), 53));
                if (!alive) break;
                const double* xb = xs + c * kChunkK + 32 * sec;
                const uint32_t cw[8] = {ca[u].x, ca[u].y, ca[u].z, ca[u].w, cb2[u].x, cb2[u].y, cb2[u].z, cb2[u].w};
                const float s0 = scale_of_raw(sq[u], sdt);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float lo, hi;
                    e4m3x2_to_f32((uint16_t)(cw[i >> 2] >> (8 * (i & 3))), lo, hi);
                    pb[i * kMaxR] = pad ? 0.0 : __dmul_rn(xb[i], (double)__fmul_rn(lo, s0));
                    pb[(i + 1) * kMaxR] = pad ? 0.0 : __dmul_rn(xb[i + 1], (double)__fmul_rn(hi, s0));
                }
                __syncwarp();
                if (lane == 0) tcdev::mbar_arrive(&full[grp]);
                const int cn = c + kChainBufs * kAhead;
                if (cn < nchunk) {
                    ca[u] = *(const uint4*)(crow + (int64_t)cn * kChunkK);
                    cb2[u] = *(const uint4*)(crow + (int64_t)cn * kChunkK + 16);
                    sq[u] = ld_scale_raw(scale, sbase + cn, sdt);
                }
            }
        }
    }
}

} /* namespace */

int launch_logit_rerank_e4m3(const void* x, int xdt, int64_t x_rs, const void* codes, int64_t code_rs,
                             const void* scale, int64_t scale_rs, int br, int sdt, const int32_t* in, int64_t in_rs,
                             int32_t* idx, int64_t idx_rs, float* val, int64_t val_rs, float* pairs, int M, int R,
                             int K, int64_t NV, int64_t voff, cudaStream_t st) {
    if (R < 1 || R > kMaxR || M < 1) return RAD_E_UNSUPPORTED;
    const size_t want = (size_t)K * sizeof(float);
    /* everything staged: x as f32, 32 head rows, their scales, a barrier; needs whole 128-K blocks and what a
     * bulk copy needs (16-byte aligned rows, a multiple of 16 bytes) */
    const size_t nblk = (size_t)(K >> 7);
    const size_t full = want + (size_t)kMaxR * K + (kMaxR * nblk + 2) * sizeof(float) + 16;
    const bool al16 = ((((uintptr_t)codes) | (uintptr_t)code_rs) & 15) == 0;
    /* the chain form: whole 128-K blocks, 16-byte aligned head rows, four chunk buffers + the row in shared memory */
    static const bool chain_off = [] { const char* e = getenv("R3D_RERANK_NO_CHAIN"); return e && *e && *e != '0'; }();
    const size_t chain_smem = (size_t)kChainBufs * kChunkDoubles * sizeof(double) + 2 * want + 2 * kChainBufs * sizeof(uint64_t);
    const bool al16c = ((((uintptr_t)codes) | (uintptr_t)code_rs) & 15) == 0;
    if (!chain_off && al16c && K >= 128 && (K & 127) == 0 && chain_smem <= 227 * 1024) {
        const int dev = tc_device();
        if (dev < 0) return RAD_E_DEVICE;
        static size_t chain_attr[kTcMaxDevices] = {};
        if (chain_smem > chain_attr[dev]) {
            if (cudaFuncSetAttribute(k_logit_rerank_chain, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)chain_smem) != cudaSuccess)
                return RAD_E_DEVICE;
            chain_attr[dev] = chain_smem;
        }
        count_launch();
        k_logit_rerank_chain<<<(unsigned)M, 32 * kChainWarps, chain_smem, st>>>(
            (const uint8_t*)x, xdt, x_rs, (const uint8_t*)codes, code_rs, scale, scale_rs, br, sdt, in, in_rs, idx, idx_rs,
            val, val_rs, pairs, R, K, NV, voff);
        return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
    }
    int mode = want <= 48 * 1024 ? 1 : 0;               /* larger rows are read through the caches */
    size_t smem = mode ? want : 0;
    if (al16 && K >= 128 && (K & 127) == 0 && full <= 227 * 1024) { mode = 2; smem = full; }
    if (smem > 48 * 1024) {
        const int dev = tc_device();
        if (dev < 0) return RAD_E_DEVICE;
        static size_t attr_set[kTcMaxDevices] = {};
        if (smem > attr_set[dev]) {
            if (cudaFuncSetAttribute(k_logit_rerank_e4m3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return RAD_E_DEVICE;
            attr_set[dev] = smem;
        }
    }
    count_launch();
    k_logit_rerank_e4m3<<<(unsigned)M, 32 * kWarps, smem, st>>>(
        (const uint8_t*)x, xdt, x_rs, (const uint8_t*)codes, code_rs, scale, scale_rs, br, sdt, in, in_rs, idx, idx_rs,
        val, val_rs, pairs, R, K, NV, voff, mode);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

int rerank_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_rr_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

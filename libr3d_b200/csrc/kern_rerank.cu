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
 * tensor core: one block of eight warps per row; the row's activations are widened to f32 once
 * into shared memory by the whole block; every warp serves four candidates at once, eight lanes
 * each: per 128-K block a lane fetches sixteen consecutive codes of its candidate's head row (one
 * 128-byte line per candidate, against the reference's one thread per candidate striding its own
 * row) with the loads of the next two blocks already in flight (a head row is touched once, so every
 * load is a DRAM round trip: unhidden they were nine tenths of the kernel's time), forms the
 * sixteen exact products, and the segment's accumulator takes the 128 products of the block in
 * ascending k through width-8 shuffles -- the same adds in the same order, four chains per FP64
 * instruction. Ragged K, unaligned heads and rows too wide for shared memory take 32-K steps of
 * four codes a lane. Thread 0 runs the selection over shared memory.
 */
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"
#include <cmath>

namespace r3d { __device__ int g_rr_status = 0; }
#define R3D_TC_STATUS_WORD ::r3d::g_rr_status
#include "tc_common.cuh"

namespace r3d {

namespace {
constexpr int kMaxR = 32;
constexpr int kWarps = 8;

__device__ __forceinline__ float ld_scale_any(const void* base, int64_t idx, int dt) {
    if (dt == RAD_F32) return ((const float*)base)[idx];
    if (dt == RAD_F16) return f16_to_f32(((const uint16_t*)base)[idx]);
    return bf16_to_f32(((const uint16_t*)base)[idx]);
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
    if (warp == 0) {
        /* without NaN scores the selection's order is a total order (value descending, lower id first,
         * earlier slot first; pads last), so a candidate's place is the count of candidates ahead of it */
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
    }
    if (threadIdx.x == 0) {
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

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
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
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

int tc_gemm2_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcg2_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} /* namespace r3d */

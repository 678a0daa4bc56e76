/* kern_topk.cu -- row_topk: exact per-row top-R (R <= 32) under the engine's one total order, value
 * descending and ties to the lower column (src/r3d_more.hip:114-118, :179-236 of libr3d, which runs
 * one block per row and re-reads the row R times).
 *
 * Here the selection is a tournament, because it serves the column-sharded LM head, whose rows are
 * 19 to 152 thousand columns wide at M = 1..16: a pass gives every warp a tile of 512 items held in
 * registers (16 per lane) and takes the tile's top R with warp shuffles only -- no shared memory, no
 * block barrier -- and passes repeat over the survivors (tiles * R of them) until one tile is left;
 * that last pass writes idx / val / pairs with `vocab_off` added. The order is total on everything
 * but NaN, so the survivors of the survivors are exactly the R the reference's rounds pick; a slot
 * that cannot be filled reports (-1, -inf) as there. A NaN's place is unspecified (in the reference
 * it depends on which thread meets it first).
 */
#include <cmath>
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

namespace {

constexpr int kTile = 512;            /* items per warp */
constexpr int kPer = kTile / 32;      /* items per lane */
constexpr int kWarps = 4;             /* warps (tiles) per block */

__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) {
    return ai >= 0 && (bi < 0 || av > bv || (av == bv && ai < bi));
}

struct TopkPass {
    const void* x; int x_dtype; int64_t x_pitch;      /* first pass: the rows themselves */
    const float* cv; const int* ci; int64_t c_pitch;  /* later passes: the previous survivors */
    int n;                                            /* items per row in this pass */
    float* ov; int* oi; int64_t o_pitch;              /* survivors out (tiles * R per row) */
    int32_t* idx; int64_t idx_pitch; float* val; int64_t val_pitch; float* pairs; int64_t pairs_pitch;
    int R; int64_t off; int last;                     /* last: one tile per row, write the outputs */
};

template <bool FIRST>
__global__ __launch_bounds__(kWarps * 32) void k_topk_pass(const TopkPass P) {
    const int lane = threadIdx.x & 31;
    const int tile = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t m = blockIdx.y;
    const int base = tile * kTile;
    if (base >= P.n) return;                          /* whole warp: no shuffle is left behind */
    float v[kPer];
    int id[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int e = base + j * 32 + lane;
        if (e < P.n) {
            if (FIRST) {
                v[j] = P.x_dtype == RAD_F32 ? ((const float*)P.x)[m * P.x_pitch + e]
                                            : bf16_to_f32(((const uint16_t*)P.x)[m * P.x_pitch + e]);
                id[j] = e;
            } else {
                v[j] = P.cv[m * P.c_pitch + e];
                id[j] = P.ci[m * P.c_pitch + e];
            }
        } else {
            v[j] = 0.0f;
            id[j] = -1;
        }
    }
    for (int r = 0; r < P.R; ++r) {
        float bv = 0.0f;
        int bi = -1, bj = -1;
#pragma unroll
        for (int j = 0; j < kPer; ++j)
            if (beats(v[j], id[j], bv, bi)) { bv = v[j]; bi = id[j]; bj = j; }
        float wv = bv;
        int wi = bi;
#pragma unroll
        for (int sh = 16; sh; sh >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, sh);
            const int oi = __shfl_xor_sync(0xffffffffu, wi, sh);
            if (beats(ov, oi, wv, wi)) { wv = ov; wi = oi; }
        }
        /* ids are unique inside a row, so exactly one lane owns the winner: it retires the item */
        if (wi >= 0 && wi == bi) {
#pragma unroll
            for (int j = 0; j < kPer; ++j)
                if (j == bj) id[j] = -1;
        }
        if (lane == 0) {
            const bool ok = wi >= 0;
            if (P.last) {
                const int32_t col = ok ? (int32_t)(wi + P.off) : -1;
                const float val = ok ? wv : -INFINITY;
                P.idx[m * P.idx_pitch + r] = col;
                P.val[m * P.val_pitch + r] = val;
                if (P.pairs) {
                    float* p = P.pairs + m * P.pairs_pitch + 2 * r;
                    p[0] = __int_as_float(col);
                    p[1] = val;
                }
            } else {
                P.ov[m * P.o_pitch + (int64_t)tile * P.R + r] = ok ? wv : -INFINITY;
                P.oi[m * P.o_pitch + (int64_t)tile * P.R + r] = ok ? wi : -1;
            }
        }
    }
}

/* plugin-owned survivor planes, two per device (ping-pong), grown on demand and never freed */
struct Survivors { float* v[2]; int* i[2]; size_t items; };
Survivors* survivors(size_t items) {
    static Survivors per_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    Survivors& S = per_dev[dev];
    if (S.items < items) {
        Survivors nw{};
        for (int k = 0; k < 2; ++k)
            if (cudaMalloc(&nw.v[k], items * sizeof(float)) != cudaSuccess ||
                cudaMalloc(&nw.i[k], items * sizeof(int)) != cudaSuccess) {
                (void)cudaGetLastError();
                return nullptr;                       /* an earlier, smaller set stays in place */
            }
        nw.items = items;
        S = nw;                                       /* the old planes may still be read by work in flight: left alone */
    }
    return &S;
}

} /* namespace */

int launch_row_topk(const void* x, int x_dtype, int64_t x_pitch, int32_t* idx, int64_t idx_pitch, float* val,
                    int64_t val_pitch, float* pairs, int64_t pairs_pitch, int M, int N, int R, int64_t off,
                    cudaStream_t st) {
    const int tiles0 = (N + kTile - 1) / kTile;
    Survivors* S = nullptr;
    if (tiles0 > 1) {
        S = survivors((size_t)M * tiles0 * R);
        if (!S) return RAD_E_DEVICE;
    }
    TopkPass P{};
    P.x = x; P.x_dtype = x_dtype; P.x_pitch = x_pitch;
    P.idx = idx; P.idx_pitch = idx_pitch; P.val = val; P.val_pitch = val_pitch;
    P.pairs = pairs; P.pairs_pitch = pairs_pitch; P.R = R; P.off = off;
    int n = N, tiles = tiles0, pass = 0;
    for (;;) {
        P.n = n; P.last = tiles == 1;
        if (!P.last) { P.ov = S->v[pass & 1]; P.oi = S->i[pass & 1]; P.o_pitch = (int64_t)tiles * R; }
        const dim3 grid((unsigned)((tiles + kWarps - 1) / kWarps), (unsigned)M);
        count_launch();
        if (pass == 0) k_topk_pass<true><<<grid, kWarps * 32, 0, st>>>(P);
        else k_topk_pass<false><<<grid, kWarps * 32, 0, st>>>(P);
        if (cudaGetLastError() != cudaSuccess) return RAD_E_DEVICE;
        if (P.last) break;
        P.cv = P.ov; P.ci = P.oi; P.c_pitch = P.o_pitch;
        n = tiles * R;
        tiles = (n + kTile - 1) / kTile;
        ++pass;
    }
    return RAD_OK;
}

} /* namespace r3d */

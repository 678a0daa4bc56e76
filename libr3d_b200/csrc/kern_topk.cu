/* kern_topk.cu -- row_topk: exact per-row top-R (R <= 32) under the engine's one total order, value
 * descending and ties to the lower column (src/r3d_more.hip:114-118, :179-236 of libr3d, which runs
 * one block per row and re-reads the row R times).
 *
 * Here the selection is a tournament, because it serves the column-sharded LM head, whose rows are
 * 19 to 152 thousand columns wide at M = 1..16. A pass gives every warp a tile of 512 items held in
 * registers (16 per lane, sorted once by each lane) and takes the tile's top R with one warp-wide
 * integer maximum and one vote per pick; the eight warps of a block leave their picks, largest
 * first, in shared memory and merge them pairwise in three steps (a bitonic half-cleaner and five
 * compare-exchange steps across the lanes per merge), so a block of 4096 items hands on R survivors. Passes repeat over the survivors until one block is
 * left (151936 columns: two launches); that last pass writes idx / val / pairs with `vocab_off`
 * added. The order is total on everything but NaN, so the survivors of the survivors are exactly
 * the R the reference's rounds pick; a slot that cannot be filled reports (-1, -inf) as there. A
 * NaN's place is unspecified (in the reference it depends on which thread meets it first).
 */
#include <cmath>
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

bool tc_pdl_on();                     /* kern_tc.cu: false under R3D_NO_PDL */

namespace {

constexpr int kTile = 512;            /* items per warp */
constexpr int kPer = kTile / 32;      /* items per lane */
constexpr int kWarps = 8;             /* warps (tiles) per block */
constexpr int kBlockItems = kTile * kWarps;
static_assert(kWarps == 8, "the block's merge is three pairwise steps");

/* An item is one 64-bit key whose unsigned order is the selection order: the high word is the
 * value mapped monotonically onto unsigned integers (-0 first folded onto +0, which the rule
 * treats as equal), the low word is 0xffffffff - column, so that of two equal values the lower
 * column is the larger key. 0 is "no item". */
__device__ __forceinline__ uint32_t ord_of(float v) {
    uint32_t u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long key_of(float v, int col) {
    return ((unsigned long long)ord_of(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)col);
}

struct TopkPass {
    const void* x; int x_dtype; int64_t x_pitch;      /* the rows: items of the first pass, values of the last */
    const unsigned long long* ck; int64_t c_pitch;    /* later passes: the previous survivors */
    int n;                                            /* items per row in this pass */
    unsigned long long* ok; int64_t o_pitch;          /* survivors out (tiles * R per row) */
    int32_t* idx; int64_t idx_pitch; float* val; int64_t val_pitch; float* pairs; int64_t pairs_pitch;
    int R; int64_t off; int last;                     /* last: one tile per row, write the outputs */
};

__device__ __forceinline__ float load_x(const TopkPass& P, int64_t m, int e) {
    return P.x_dtype == RAD_F32 ? ((const float*)P.x)[m * P.x_pitch + e]
                                : bf16_to_f32(((const uint16_t*)P.x)[m * P.x_pitch + e]);
}

/* each lane sorts its NP keys, largest first (bitonic network, every index a constant) */
template <int NP>
__device__ __forceinline__ void sort_desc(unsigned long long (&k)[NP]) {
#pragma unroll
    for (int kk = 2; kk <= NP; kk <<= 1)
#pragma unroll
        for (int jj = kk >> 1; jj > 0; jj >>= 1)
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int l = i ^ jj;
                if (l > i) {
                    const bool desc = (i & kk) == 0;
                    const unsigned long long a = k[i], b = k[l];
                    const bool sw = desc ? a < b : a > b;
                    k[i] = sw ? b : a;
                    k[l] = sw ? a : b;
                }
            }
}

/* One warp's tournament over 32 sorted lists of NP keys. The lists go to shared memory ([item][lane]:
 * no bank conflicts); a lane keeps only its head in a register and fetches the next item when it
 * wins. R rounds: the largest head value of the warp (one warp-wide integer maximum); of the lanes
 * that hold it the lowest wins (one vote), because items lie in the warp's range in ascending column
 * order wherever their values are equal -- in the rows themselves by construction, among a block's
 * picks because its warps cover ascending column ranges and each lists equal values in ascending
 * column, and among survivors because blocks do the same. The winner (lane 0 when nothing is left)
 * hands the pick to emit(r, ok, key) and pops it. */
template <int NP, typename Emit>
__device__ __forceinline__ void tournament(unsigned long long (&k)[NP], unsigned long long (*sk)[32],
                                           const int lane, const int R, Emit emit) {
#pragma unroll
    for (int j = 0; j < NP; ++j) sk[j][lane] = k[j];
    /* head and its successor live in registers and the round has no branch around the pop: a win
     * moves the successor up and asks shared memory for the one after, off the critical path */
    unsigned long long head = k[0], next = NP > 1 ? k[1] : 0ull;
    int h = 0;
    for (int r = 0; r < R; ++r) {
        const uint32_t hi = (uint32_t)(head >> 32);
        const uint32_t vmax = __reduce_max_sync(0xffffffffu, hi);
        const bool ok = vmax != 0u;
        const uint32_t holders = __ballot_sync(0xffffffffu, ok && hi == vmax);
        const bool win = lane == (ok ? __ffs(holders) - 1 : 0);
        if (win) emit(r, ok, head);
        const bool pop = win && ok;
        h += pop ? 1 : 0;
        const unsigned long long after = sk[h + 1 < NP ? h + 1 : NP - 1][lane];
        head = pop ? next : head;
        next = pop ? (h + 1 < NP ? after : 0ull) : next;
    }
}

template <bool FIRST>
__global__ __launch_bounds__(kWarps * 32) void k_topk_pass(const TopkPass P) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int64_t m = blockIdx.y;
    const int block0 = blockIdx.x * kBlockItems;
    const int base = block0 + wib * kTile;
    /* passes are launched with programmatic stream serialisation: the next pass may take its
     * place on the machine now, and this one reads nothing before its predecessor has finished */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ unsigned long long s_k[kWarps][kPer][32];
    __shared__ unsigned long long s_pick[kWarps][32];           /* a warp's picks, largest first, zeros behind */
    __shared__ unsigned long long s_m1[kWarps / 2][32], s_m2[kWarps / 4][32];
    __shared__ int s_col[32];
    /* a block whose items fit one warp's tile needs no merge: that warp's picks are the block's */
    const bool one_tile = P.n - block0 <= kTile;
    if (one_tile && wib != 0) return;
    auto hand_on = [&](int r, bool ok, unsigned long long key) {
        if (P.last) s_col[r] = ok ? (int)(0xffffffffu - (uint32_t)key) : -1;
        else P.ok[m * P.o_pitch + (int64_t)blockIdx.x * P.R + r] = ok ? key : 0ull;
    };
    {
        unsigned long long k[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int e = base + lane * kPer + j;            /* a lane owns 16 neighbouring items */
            k[j] = 0ull;
            if (e < P.n) k[j] = FIRST ? key_of(load_x(P, m, e), e) : P.ck[m * P.c_pitch + e];
        }
        sort_desc<kPer>(k);
        if (one_tile) {
            tournament<kPer>(k, s_k[0], lane, P.R, hand_on);
        } else {
            s_pick[wib][lane] = 0ull;
            __syncwarp();
            tournament<kPer>(k, s_k[wib], lane, P.R,
                             [&](int r, bool ok, unsigned long long key) { s_pick[wib][r] = ok ? key : 0ull; });
        }
    }
    if (!one_tile) {
        /* the eight sorted lists merge pairwise in three steps. Keys are distinct (the column is
         * part of the key), so plain 64-bit comparisons give the selection order. Two lists of 32,
         * largest first: max(X[i], Y[31 - i]) over i holds the 32 largest of both as a bitonic
         * sequence, which five compare-exchange steps across the lanes sort. */
        auto merge2 = [&](const unsigned long long* x, const unsigned long long* y) {
            const unsigned long long a = x[lane], b = y[31 - lane];
            unsigned long long z = a > b ? a : b;
#pragma unroll
            for (int s2 = 16; s2; s2 >>= 1) {
                const unsigned long long o = __shfl_xor_sync(0xffffffffu, z, s2);
                const bool up = (lane & s2) == 0;           /* the lower lane of a pair keeps the larger key */
                z = (up == (z > o)) ? z : o;
            }
            return z;
        };
        __syncthreads();
        if (wib < kWarps / 2) s_m1[wib][lane] = merge2(s_pick[2 * wib], s_pick[2 * wib + 1]);
        __syncthreads();
        if (wib < kWarps / 4) s_m2[wib][lane] = merge2(s_m1[2 * wib], s_m1[2 * wib + 1]);
        __syncthreads();
        if (wib != 0) return;
        const unsigned long long z = merge2(s_m2[0], s_m2[1]);
        if (lane < P.R) hand_on(lane, z != 0ull, z);
    }
    if (P.last) {
        /* lane r writes pick r; the value is re-read from the row (a zero keeps its sign) */
        __syncwarp();
        if (lane < P.R) {
            const int col = s_col[lane];
            const int32_t out_col = col >= 0 ? (int32_t)(col + P.off) : -1;
            const float out_val = (col >= 0 && (P.val || P.pairs)) ? load_x(P, m, col) : -INFINITY;
            P.idx[m * P.idx_pitch + lane] = out_col;
            if (P.val) P.val[m * P.val_pitch + lane] = out_val;
            if (P.pairs) {
                float* p = P.pairs + m * P.pairs_pitch + 2 * lane;
                p[0] = __int_as_float(out_col);
                p[1] = out_val;
            }
        }
    }
}

/* plugin-owned survivor planes, two per device (ping-pong), grown on demand and never freed */
struct Survivors { unsigned long long* k[2]; size_t items; };
Survivors* survivors(size_t items) {
    static Survivors per_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    Survivors& S = per_dev[dev];
    if (S.items < items) {
        Survivors nw{};
        for (int b = 0; b < 2; ++b)
            if (cudaMalloc(&nw.k[b], items * sizeof(unsigned long long)) != cudaSuccess) {
                (void)cudaGetLastError();
                return nullptr;                       /* an earlier, smaller set stays in place */
            }
        nw.items = items;
        S = nw;                                       /* the old planes may still be read by work in flight: left alone */
    }
    return &S;
}

} /* namespace */

/* bytes of the two survivor planes a call needs (0 when the row fits one block): what the rows' scratch
 * hooks ask the engine for */
int64_t row_topk_scratch_bytes(int64_t M, int64_t N, int64_t R) {
    const int64_t tiles0 = (N + kBlockItems - 1) / kBlockItems;
    return tiles0 > 1 ? 2 * M * tiles0 * R * (int64_t)sizeof(unsigned long long) : 0;
}

int launch_row_topk(const void* x, int x_dtype, int64_t x_pitch, int32_t* idx, int64_t idx_pitch, float* val,
                    int64_t val_pitch, float* pairs, int64_t pairs_pitch, int M, int N, int R, int64_t off,
                    cudaStream_t st, void* scratch, int64_t scratch_bytes) {
    const int tiles0 = (N + kBlockItems - 1) / kBlockItems;          /* blocks of the first pass */
    Survivors* S = nullptr;
    Survivors arena{};
    if (tiles0 > 1) {
        /* the launch arena when the engine provides one (the rows declare a scratch hook: nothing is
         * allocated then); the plugin's own planes otherwise, grown on first use */
        const size_t items = (size_t)M * tiles0 * R;
        if (scratch && scratch_bytes >= row_topk_scratch_bytes(M, N, R) && (((uintptr_t)scratch) & 7) == 0) {
            arena.k[0] = (unsigned long long*)scratch; arena.k[1] = arena.k[0] + items; arena.items = items;
            S = &arena;
        } else {
            S = survivors(items);
        }
        if (!S) return RAD_E_DEVICE;
    }
    TopkPass P{};
    P.x = x; P.x_dtype = x_dtype; P.x_pitch = x_pitch;
    P.idx = idx; P.idx_pitch = idx_pitch; P.val = val; P.val_pitch = val_pitch;
    P.pairs = pairs; P.pairs_pitch = pairs_pitch; P.R = R; P.off = off;
    int n = N, tiles = tiles0, pass = 0;
    for (;;) {
        P.n = n; P.last = tiles == 1;
        if (!P.last) { P.ok = S->k[pass & 1]; P.o_pitch = (int64_t)tiles * R; }
        const dim3 grid((unsigned)tiles, (unsigned)M);
        count_launch();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid; cfg.blockDim = dim3(kWarps * 32); cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = tc_pdl_on() ? 1 : 0;
        const cudaError_t e = pass == 0 ? cudaLaunchKernelEx(&cfg, k_topk_pass<true>, P)
                                        : cudaLaunchKernelEx(&cfg, k_topk_pass<false>, P);
        if (e != cudaSuccess) return RAD_E_DEVICE;
        if (P.last) break;
        P.ck = P.ok; P.c_pitch = P.o_pitch;
        n = tiles * R;
        tiles = (n + kBlockItems - 1) / kBlockItems;
        ++pass;
    }
    return RAD_OK;
}

} /* namespace r3d */

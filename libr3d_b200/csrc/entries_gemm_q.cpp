/* entries_gemm_q.cpp -- the gemm_nt_q row entries at the fp8a8 and mxfp4a8 encodings.
 *
 * Host C++ only. Each entry reads its RadArgs the way libr3d's does -- operands by schema
 * position (a, a_scale, b, b_scale, y, a_sum?, b_ref?), M from numel(y)/N and never from
 * the M parameter, scale grids from tensor shapes -- refuses with the same status codes in
 * the same precedence, and hands a validated plan to the launch layer (r3d_b200_gemm_*).
 *   fp8a8    src/r3d_gemm_fp8a8.hip:852-924 (plan), :1055-1130 (entries)
 *   mxfp4a8  src/r3d_gemm_mxfp4.hip:1521-1582 (plan), :1587-1611, :1715-1772 (entries)
 *
 * Two documented supersets of the reference's fp8a8 contract, for the per-channel /
 * per-token checkpoints: b_scale may be f32, and either scale grid may have a single
 * column (one scale for the whole of K, applied at every 128-of-K flush).
 */
#include <cstdio>
#include <vector>
#include <cuda_runtime.h>
#include "entry_util.h"
#include "r3d_b200.h"

using namespace r3d;

namespace {

/* ------------------------------------------------------------------ fp8a8 plan */
int plan_fp8a8(const RadArgs* a, const RadTensor* A, const RadTensor* AS, const RadTensor* B,
               const RadTensor* BS, const RadTensor* Y, long long M, long long Nparam,
               R3dGemmQ* q) {
    const char* enc = rad_args_gets(a, "dtype");
    if (!enc || strcmp(enc, "fp8a8") != 0) return RAD_E_UNSUPPORTED;
    long long part = 0;
    if (rad_args_geti(a, "pb1", &part) && part > 0) return RAD_E_UNSUPPORTED;  /* e2m1-only */
    if (rad_args_geti(a, "pb2", &part) && part > 0) return RAD_E_UNSUPPORTED;
    if (A->dtype != RAD_F8E4M3 || B->dtype != RAD_F8E4M3 || AS->dtype != RAD_F32 ||
        (BS->dtype != RAD_BF16 && BS->dtype != RAD_F32))
        return RAD_E_UNSUPPORTED;

    long long N = 0, K = 0;
    if (!rad_args_geti(a, "N", &N) || !rad_args_geti(a, "K", &K)) return RAD_E_SHAPE;
    if (N <= 0 || K <= 0) return RAD_E_SHAPE;
    if (K % 128) return RAD_E_UNSUPPORTED;            /* a scale block must close */
    if (M <= 0) return RAD_E_SHAPE;
    if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return RAD_E_SHAPE;
    if (rad_tensor_numel(A) < M * K || rad_tensor_numel(B) < N * K) return RAD_E_SHAPE;

    if (BS->rank != 2 || BS->stride[1] != 1) return RAD_E_UNSUPPORTED;
    if (AS->rank != 2 || AS->stride[1] != 1 || (long long)AS->shape[0] < M)
        return RAD_E_UNSUPPORTED;
    const int64_t bs_cols = BS->shape[1], as_cols = AS->shape[1];
    const int64_t nchunk = K / 128;
    /* the grid the bytes describe: 128 of K per column, or (superset) one column */
    const bool b_whole = bs_cols == 1 && nchunk > 1, a_whole = as_cols == 1 && nchunk > 1;
    if (!b_whole && grid_block(K, bs_cols) != 128) return RAD_E_UNSUPPORTED;
    if (!a_whole && grid_block(K, as_cols) != 128) return RAD_E_UNSUPPORTED;
    if ((!b_whole && bs_cols != nchunk) || (!a_whole && as_cols != nchunk)) return RAD_E_SHAPE;
    if (rad_tensor_numel(AS) < M * as_cols) return RAD_E_SHAPE;

    int rblk;
    if ((long long)BS->shape[0] >= N) {
        if ((long long)BS->shape[0] != N) return RAD_E_SHAPE;
        rblk = 1;                                      /* one scale row per weight row */
    } else {
        if (grid_block(N, BS->shape[0]) != 128 || (long long)BS->shape[0] != (N + 127) / 128)
            return RAD_E_UNSUPPORTED;
        rblk = 128;                                    /* the 128x128 checkpoint grid */
    }
    if (rad_tensor_numel(BS) < (rblk > 1 ? (N + 127) / 128 : N) * bs_cols) return RAD_E_SHAPE;

    long long gp = 0;
    if (rad_args_geti(a, "group", &gp) && gp > 0 && gp != 128 &&
        !((a_whole || b_whole) && gp == K))
        return RAD_E_SHAPE;

    if (!inner_contiguous(A) || !inner_contiguous(B)) return RAD_E_STRIDE;

    q->a = A->data; q->a_scale = (const float*)AS->data; q->b = B->data; q->b_scale = BS->data;
    q->y = Y->data;
    q->m = (int32_t)M; q->n = (int32_t)N; q->k = (int32_t)K;
    q->as_cols = (int32_t)as_cols; q->bs_cols = (int32_t)bs_cols;
    q->rblk = rblk; q->bs_dtype = (int32_t)BS->dtype;
    q->a_pitch = row_pitch(A, K); q->b_pitch = row_pitch(B, K);
    q->y_pitch = row_pitch(Y, Nparam);
    q->as_pitch = row_pitch(AS, as_cols); q->bs_pitch = row_pitch(BS, bs_cols);
    q->arm = R3D_ARM_AUTO;
    return RAD_OK;
}

int run_fp8a8(const RadArgs* a, RadStream s, bool decode_band) {
    static const bool off_all = env_present("R3D_NO_FP8A8");
    static const bool off_dec = env_present("R3D_NO_FP8_DEC");
    if (off_all || (decode_band && off_dec)) return RAD_E_UNSUPPORTED;

    const RadTensor* A = rad_arg_in(a, 0);
    const RadTensor* AS = rad_arg_in(a, 1);
    const RadTensor* B = rad_arg_in(a, 2);
    const RadTensor* BS = rad_arg_in(a, 3);
    const RadTensor* Y = rad_arg_in(a, 4);
    if (!A || !AS || !B || !BS || !Y) return RAD_E_UNSUPPORTED;
    if (rad_arg_in(a, 5) || rad_arg_in(a, 6)) return RAD_E_UNSUPPORTED;   /* a_sum, b_ref */
    if (Y->dtype != RAD_BF16) return RAD_E_UNSUPPORTED;

    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0) return RAD_E_SHAPE;
    const long long Yn = rad_tensor_numel(Y);
    if (Yn <= 0 || Yn % N) return RAD_E_SHAPE;
    if (decode_band && Yn / N > 8) return RAD_E_UNSUPPORTED;              /* the band's bound */
    if (!inner_contiguous(Y)) return RAD_E_STRIDE;

    R3dGemmQ q{};
    const int rc = plan_fp8a8(a, A, AS, B, BS, Y, Yn / N, N, &q);
    if (rc != RAD_OK) return rc;
    /* the decode row keeps the reference's promise that a weight plane off the 4-byte grid
     * resolves past it (src/r3d_gemm_fp8a8.hip:1127) */
    if (decode_band && ((q.b_pitch % 4) != 0 || (((uintptr_t)q.b) & 3) != 0))
        return RAD_E_UNSUPPORTED;
    return r3d_b200_gemm_fp8a8(&q, (void*)s);
}

/* ------------------------------------------------------------------ mxfp4a8 plan */
int plan_mxfp4a8(const RadArgs* a, const RadTensor* A, const RadTensor* AS, const RadTensor* B,
                 const RadTensor* BS, const RadTensor* Y, long long M, long long N,
                 R3dGemmQ* q) {
    const char* enc = rad_args_gets(a, "dtype");
    if (!enc || strcmp(enc, "mxfp4a8") != 0) return RAD_E_UNSUPPORTED;
    long long part = 0;
    if (rad_args_geti(a, "pb1", &part) && part > 0) return RAD_E_UNSUPPORTED;
    if (rad_args_geti(a, "pb2", &part) && part > 0) return RAD_E_UNSUPPORTED;
    if (A->dtype != RAD_F8E4M3 || B->dtype != RAD_FP4E2M1 || Y->dtype != RAD_BF16 ||
        AS->dtype != RAD_F32 || (BS->dtype != RAD_E8M0 && BS->dtype != RAD_U8))
        return RAD_E_UNSUPPORTED;

    long long K = 0;
    if (!rad_args_geti(a, "K", &K)) return RAD_E_SHAPE;
    if (N <= 0 || K <= 0 || M <= 0) return RAD_E_SHAPE;
    if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return RAD_E_SHAPE;
    if (rad_tensor_numel(A) < M * K || rad_tensor_numel(B) < N * K) return RAD_E_SHAPE;

    if (BS->rank != 2 || BS->stride[1] != 1 || (long long)BS->shape[0] < N)
        return RAD_E_UNSUPPORTED;
    if (AS->rank != 2 || AS->stride[1] != 1 || (long long)AS->shape[0] < M)
        return RAD_E_UNSUPPORTED;
    const int64_t bs_cols = BS->shape[1], as_cols = AS->shape[1];
    if (grid_block(K, bs_cols) != 32 || grid_block(K, as_cols) != 128) return RAD_E_UNSUPPORTED;
    if (bs_cols != (K + 31) / 32 || as_cols != (K + 127) / 128) return RAD_E_UNSUPPORTED;
    if (rad_tensor_numel(AS) < M * as_cols) return RAD_E_SHAPE;

    if (!inner_contiguous(A) || !inner_contiguous(B) || !inner_contiguous(Y)) return RAD_E_STRIDE;
    if ((K & 1) || row_pitch(B, K) != K) return RAD_E_STRIDE;     /* rows byte-packed exactly */

    q->a = A->data; q->a_scale = (const float*)AS->data; q->b = B->data; q->b_scale = BS->data;
    q->y = Y->data;
    q->m = (int32_t)M; q->n = (int32_t)N; q->k = (int32_t)K;
    q->as_cols = (int32_t)as_cols; q->bs_cols = (int32_t)bs_cols;
    q->rblk = 1; q->bs_dtype = RAD_E8M0;
    q->a_pitch = row_pitch(A, K); q->b_pitch = K / 2;
    q->y_pitch = row_pitch(Y, N);
    q->as_pitch = row_pitch(AS, as_cols); q->bs_pitch = row_pitch(BS, bs_cols);
    q->arm = R3D_ARM_AUTO;
    return RAD_OK;
}

/* ------------------------------------------------------------------ mxfp4mx8 plan
 * The mxfp4a8 plan with the activation's scale grid changed: E8M0 bytes, one per 32 of K. The
 * same refusal order as the mxfp4a8 entry (src/r3d_gemm_mxfp4.hip:1521-1582 of libr3d), which has no
 * such spelling itself. */
int plan_mxfp4mx8(const RadArgs* a, const RadTensor* A, const RadTensor* AS, const RadTensor* B,
                  const RadTensor* BS, const RadTensor* Y, long long M, long long N, R3dGemmQ* q) {
    const char* enc = rad_args_gets(a, "dtype");
    if (!enc || strcmp(enc, "mxfp4mx8") != 0) return RAD_E_UNSUPPORTED;
    long long part = 0;
    if (rad_args_geti(a, "pb1", &part) && part > 0) return RAD_E_UNSUPPORTED;
    if (rad_args_geti(a, "pb2", &part) && part > 0) return RAD_E_UNSUPPORTED;
    if (A->dtype != RAD_F8E4M3 || B->dtype != RAD_FP4E2M1 || Y->dtype != RAD_BF16 ||
        (AS->dtype != RAD_E8M0 && AS->dtype != RAD_U8) || (BS->dtype != RAD_E8M0 && BS->dtype != RAD_U8))
        return RAD_E_UNSUPPORTED;
    long long K = 0;
    if (!rad_args_geti(a, "K", &K)) return RAD_E_SHAPE;
    if (N <= 0 || K <= 0 || M <= 0) return RAD_E_SHAPE;
    if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return RAD_E_SHAPE;
    if (rad_tensor_numel(A) < M * K || rad_tensor_numel(B) < N * K) return RAD_E_SHAPE;
    if (BS->rank != 2 || BS->stride[1] != 1 || (long long)BS->shape[0] < N) return RAD_E_UNSUPPORTED;
    if (AS->rank != 2 || AS->stride[1] != 1 || (long long)AS->shape[0] < M) return RAD_E_UNSUPPORTED;
    const int64_t bs_cols = BS->shape[1], as_cols = AS->shape[1];
    if (grid_block(K, bs_cols) != 32 || grid_block(K, as_cols) != 32) return RAD_E_UNSUPPORTED;
    if (bs_cols != (K + 31) / 32 || as_cols != (K + 31) / 32) return RAD_E_UNSUPPORTED;
    if (rad_tensor_numel(AS) < M * as_cols) return RAD_E_SHAPE;
    if (!inner_contiguous(A) || !inner_contiguous(B) || !inner_contiguous(Y)) return RAD_E_STRIDE;
    if ((K & 1) || row_pitch(B, K) != K) return RAD_E_STRIDE;
    q->a = A->data; q->a_scale = (const float*)AS->data; q->b = B->data; q->b_scale = BS->data;
    q->y = Y->data;
    q->m = (int32_t)M; q->n = (int32_t)N; q->k = (int32_t)K;
    q->as_cols = (int32_t)as_cols; q->bs_cols = (int32_t)bs_cols;
    q->rblk = 1; q->bs_dtype = RAD_E8M0;
    q->a_pitch = row_pitch(A, K); q->b_pitch = K / 2;
    q->y_pitch = row_pitch(Y, N);
    q->as_pitch = row_pitch(AS, as_cols); q->bs_pitch = row_pitch(BS, bs_cols);
    q->arm = R3D_ARM_AUTO;
    return RAD_OK;
}

/* Immortal per-K scratch of the int8 arm: pointers must never move once handed to a
 * launch, because the engine may record a pass and replay it with the recorded arguments
 * (src/r3d_gemm_mxfp4.hip:1841-1849). One buffer pair per distinct K, never freed. */
struct Q8xScratch { long long k; int8_t* x8; float* sg; };

bool q8x_scratch_for(long long K, int8_t** x8, float** sg, cudaStream_t st) {
    static std::vector<Q8xScratch> pool;
    static bool dead = false;
    for (const Q8xScratch& e : pool) if (e.k == K) { *x8 = e.x8; *sg = e.sg; return true; }
    if (dead) return false;
    /* a first call for this K that arrives while its stream is being recorded cannot allocate (the
     * allocation would invalidate the recording): this call rides the fp32 walk, the next call
     * outside a recording builds the scratch */
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    if (cap != cudaStreamCaptureStatusNone) return false;
    /* host-side fault injection for the fallback test: makes the allocator "fail" */
    static const bool inject = env_present("R3D_Q8X_FAIL_ALLOC");
    int8_t* nx = nullptr; float* ns = nullptr;
    if (!inject && cudaMalloc((void**)&nx, (size_t)(8 * K)) == cudaSuccess &&
        cudaMalloc((void**)&ns, (size_t)(8 * (K >> 5)) * sizeof(float)) == cudaSuccess) {
        pool.push_back(Q8xScratch{K, nx, ns});
        *x8 = nx; *sg = ns;
        return true;
    }
    if (nx) (void)cudaFree(nx);
    (void)cudaGetLastError();
    dead = true;
    fprintf(stderr, "libr3d_b200: mxfp4 q8x scratch unavailable -- the fp32 walk keeps this band\n");
    return false;
}

int run_mxfp4_decode(const RadArgs* a, RadStream s, bool q8x_row) {
    static const bool off = env_present("R3D_NO_MXFP4") || env_present("R3D_NO_FP4_DEC");
    if (off) return RAD_E_UNSUPPORTED;
    if (q8x_row && r3d_mxfp4_q8x_off()) return RAD_E_UNSUPPORTED;  /* backstop of the gate */

    const RadTensor* A = rad_arg_in(a, 0);
    const RadTensor* AS = rad_arg_in(a, 1);
    const RadTensor* B = rad_arg_in(a, 2);
    const RadTensor* BS = rad_arg_in(a, 3);
    const RadTensor* Y = rad_arg_in(a, 4);
    if (!A || !AS || !B || !BS || !Y) return RAD_E_UNSUPPORTED;
    if (rad_arg_in(a, 5)) return RAD_E_UNSUPPORTED;                 /* a_sum; b_ref is ignored */
    if (Y->dtype != RAD_BF16) return RAD_E_UNSUPPORTED;

    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0) return RAD_E_SHAPE;
    const long long Yn = rad_tensor_numel(Y);
    if (Yn <= 0 || Yn % N) return RAD_E_SHAPE;
    if (Yn / N > 8) return RAD_E_UNSUPPORTED;

    R3dGemmQ q{};
    const int rc = plan_mxfp4a8(a, A, AS, B, BS, Y, Yn / N, N, &q);
    if (rc != RAD_OK) return rc;
    if (q.k % 128) return RAD_E_UNSUPPORTED;
    if ((q.b_pitch % 4) != 0 || (((uintptr_t)q.b) & 3) != 0) return RAD_E_UNSUPPORTED;

    if (q8x_row && (q.k & 255) == 0 && q.k <= (1 << 20)) {
        int8_t* x8 = nullptr; float* sg = nullptr;
        if (q8x_scratch_for(q.k, &x8, &sg, (cudaStream_t)(uintptr_t)s)) {
            /* walk lever, three states like the reference's R3D_Q8X_LMAP
             * (src/r3d_gemm_mxfp4.hip:2065-2076): "0" tree walk always, "2" lane map always,
             * default lane map for 4 or more tokens */
            static const int lmap = [] {
                const char* e = getenv("R3D_Q8X_LMAP");
                return (e && e[0] == '0') ? 0 : (e && e[0] == '2') ? 2 : 1; }();
            const int walk = (lmap == 2 || (lmap == 1 && q.m > 2)) ? 1 : 0;
            const int qrc = r3d_b200_gemm_mxfp4a8_q8x(&q, x8, sg, walk, (void*)s);
            if (qrc == RAD_OK) return RAD_OK;
            fprintf(stderr, "libr3d_b200: mxfp4 q8x arm launch failed (%d); the fp32 walk takes "
                            "this launch\n", qrc);
        }
        /* fall through: never a refusal -- the engine chose this row at declare time */
    }
    return r3d_b200_gemm_mxfp4a8(&q, (void*)s);
}

} /* namespace */

extern "C" {

int r3d_rad_gemm_nt_q_fp8(const RadArgs* a, RadStream s) { return run_fp8a8(a, s, false); }
int r3d_rad_gemm_nt_q_fp8_decode(const RadArgs* a, RadStream s) { return run_fp8a8(a, s, true); }

int r3d_rad_gemm_nt_q(const RadArgs* a, RadStream s) {
    static const bool off = env_present("R3D_NO_MXFP4");
    if (off) return RAD_E_UNSUPPORTED;
    const RadTensor* A = rad_arg_in(a, 0);
    const RadTensor* AS = rad_arg_in(a, 1);
    const RadTensor* B = rad_arg_in(a, 2);
    const RadTensor* BS = rad_arg_in(a, 3);
    const RadTensor* Y = rad_arg_in(a, 4);
    if (!A || !AS || !B || !BS || !Y) return RAD_E_UNSUPPORTED;
    if (rad_arg_in(a, 5)) return RAD_E_UNSUPPORTED;                 /* a_sum */
    if (Y->dtype != RAD_BF16) return RAD_E_UNSUPPORTED;
    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0) return RAD_E_SHAPE;
    const long long Yn = rad_tensor_numel(Y);
    if (Yn <= 0 || Yn % N) return RAD_E_SHAPE;
    R3dGemmQ q{};
    const int rc = plan_mxfp4a8(a, A, AS, B, BS, Y, Yn / N, N, &q);
    if (rc != RAD_OK) return rc;
    return r3d_b200_gemm_mxfp4a8(&q, (void*)s);
}

int r3d_rad_gemm_nt_q_mx8(const RadArgs* a, RadStream s) {
    static const bool off = env_present("R3D_NO_MXFP4");
    if (off) return RAD_E_UNSUPPORTED;
    const RadTensor* A = rad_arg_in(a, 0);
    const RadTensor* AS = rad_arg_in(a, 1);
    const RadTensor* B = rad_arg_in(a, 2);
    const RadTensor* BS = rad_arg_in(a, 3);
    const RadTensor* Y = rad_arg_in(a, 4);
    if (!A || !AS || !B || !BS || !Y) return RAD_E_UNSUPPORTED;
    if (rad_arg_in(a, 5)) return RAD_E_UNSUPPORTED;                 /* a_sum; b_ref is ignored */
    if (Y->dtype != RAD_BF16) return RAD_E_UNSUPPORTED;
    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0) return RAD_E_SHAPE;
    const long long Yn = rad_tensor_numel(Y);
    if (Yn <= 0 || Yn % N) return RAD_E_SHAPE;
    R3dGemmQ q{};
    const int rc = plan_mxfp4mx8(a, A, AS, B, BS, Y, Yn / N, N, &q);
    if (rc != RAD_OK) return rc;
    return r3d_b200_gemm_mxfp4mx8(&q, (void*)s);
}

int r3d_rad_gemm_nt_q_mxfp4_decode(const RadArgs* a, RadStream s) {
    return run_mxfp4_decode(a, s, false);
}
int r3d_rad_gemm_nt_q_mxfp4_decode_q8x(const RadArgs* a, RadStream s) {
    return run_mxfp4_decode(a, s, true);
}

/* gemm_nt_q_gated @ fp8a8 (src/r3d_gemm_fp8a8.hip:1167-1253 of libr3d): operands a, a_scale, b, b_scale,
 * q (e4m3 [M, n]), scale (f32 [M, n/group]), out_bf16 (optional, bf16 or f32), a_sum (refused). The
 * [2n, K] gate_up weight's product lands as bf16 [M, 2n] in the launch scratch, then the gated
 * quantiser reads it: byte-identical to gemm_nt_q followed by gated_quant_fp8, because it is that
 * pair. Wide projections (no K split, n a multiple of 128, group 128) at M <= 8 run as ONE launch instead: the
 * tcgen05 decode kernel takes a gate tile and its up tile in a cluster of two and closes with the
 * quantiser in its epilogue -- the same accumulation and the same statements, so the same bytes. M = numel(q) / n; `act` is required; the arena (64 * N * 2 bytes, the scratch hook) is
 * checked, never overrun. */
int r3d_rad_gemm_nt_q_gated_fp8(const RadArgs* a, RadStream s) {
    static const bool off = env_present("R3D_NO_FP8A8");
    if (off) return RAD_E_UNSUPPORTED;
    const RadTensor* A = rad_arg_in(a, 0);
    const RadTensor* AS = rad_arg_in(a, 1);
    const RadTensor* B = rad_arg_in(a, 2);
    const RadTensor* BS = rad_arg_in(a, 3);
    const RadTensor* Q = rad_arg_in(a, 4);
    const RadTensor* SC = rad_arg_in(a, 5);
    const RadTensor* OB = rad_arg_in(a, 6);
    if (!A || !AS || !B || !BS || !Q || !SC) return RAD_E_UNSUPPORTED;
    if (rad_arg_in(a, 7)) return RAD_E_UNSUPPORTED;                       /* a_sum */
    if (Q->dtype != RAD_F8E4M3 || SC->dtype != RAD_F32) return RAD_E_UNSUPPORTED;
    if (OB && OB->dtype != RAD_BF16 && OB->dtype != RAD_F32) return RAD_E_UNSUPPORTED;
    const char* act = rad_args_gets(a, "act");
    if (!act) return RAD_E_UNSUPPORTED;
    const int silu = strcmp(act, "sigmoid") != 0;
    if (silu && strcmp(act, "silu") != 0) return RAD_E_UNSUPPORTED;

    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0 || (N & 1)) return RAD_E_SHAPE;
    const long long n = N / 2;
    long long g = 0;
    if (!rad_args_geti(a, "group", &g) || g <= 0) g = n;
    if (g > n) g = n;
    const long long ngrp = (n + g - 1) / g;
    const long long Qn = rad_tensor_numel(Q);
    if (Qn <= 0 || Qn % n) return RAD_E_SHAPE;
    const long long M = Qn / n;
    if (rad_tensor_numel(SC) < M * ngrp) return RAD_E_SHAPE;
    if (OB && rad_tensor_numel(OB) < M * n) return RAD_E_SHAPE;

    const int64_t need = M * N * (int64_t)sizeof(uint16_t);
    RadTensor plane{};                                  /* the gate_up product, bf16 [M, N] in the arena */
    plane.data = a->scratch; plane.dtype = RAD_BF16; plane.rank = 2;
    plane.shape[0] = M; plane.shape[1] = N; plane.stride[0] = N; plane.stride[1] = 1;
    R3dGemmQ q{};
    /* the plain row's plan on the same operands; its "group" rule (128 of K) is the gated row's
     * constraint too, while `g` above is the quantiser's own group over n */
    const int rc = plan_fp8a8(a, A, AS, B, BS, &plane, M, N, &q);
    if (rc != RAD_OK) return rc;
    if (!a->scratch || a->scratch_bytes < need) return RAD_E_UNSUPPORTED;
    if (!inner_contiguous(Q) || !inner_contiguous(SC) || (OB && !inner_contiguous(OB))) return RAD_E_STRIDE;

    /* one launch where the fused kernel gives the pair's bytes (group 128 = one gate tile a quantiser group)
     * and is the faster of the two: up to eight tokens (measured at 2n = 27648, K = 5120: 26.1 / 27.6 / 29.4 us
     * against 29.1 / 29.6 / 30.4 for M = 1 / 4 / 8; at sixteen tokens the exponentials in the kernel's tail
     * cost more than the second launch saves, 33.3 against 32.2); the pair otherwise */
    if (g == 128 && M <= 8) {
        const int rf = r3d_b200_gemm_fp8a8_gated(&q, Q->data, row_pitch(Q, n), (float*)SC->data, row_pitch(SC, ngrp),
                                                 OB ? OB->data : nullptr, OB ? (int32_t)OB->dtype : RAD_BF16,
                                                 OB ? row_pitch(OB, n) : 0, silu, (void*)s);
        if (rf != RAD_E_UNSUPPORTED) return rf;
    }
    const int rg = r3d_b200_gemm_fp8a8(&q, (void*)s);
    if (rg != RAD_OK) return rg;
    return r3d_b200_gated_quant_fp8(a->scratch, N, Q->data, row_pitch(Q, n), (float*)SC->data, row_pitch(SC, ngrp),
                                    OB ? OB->data : nullptr, OB ? (int32_t)OB->dtype : RAD_BF16,
                                    OB ? row_pitch(OB, n) : 0, (int32_t)M, (int32_t)n, (int32_t)g, silu, (void*)s);
}

/* the arena of the fused row: the [M, N] bf16 plane at the band's M bound (M <= 64) */
int64_t r3d_rad_gemm_nt_q_gated_fp8_scratch(const RadArgs* a) {
    long long N = 0;
    if (!rad_args_geti(a, "N", &N) || N <= 0 || N > (1LL << 34)) return 0;
    return 64 * N * (int64_t)sizeof(uint16_t);
}

bool r3d_mxfp4_q8x_off(void) {
    static const bool off = env_is_zero("R3D_MXFP4_Q8X");
    return off;
}

} /* extern "C" */

/* entries_band.cpp -- the activation producers that sit in front of the quantised matmul bands:
 * quant_act_fp8, gated_quant_fp8 and rmsnorm_quant_fp8, as kernel rows of their own.
 *
 * Host C++ only. Operands are read by schema position, every refusal carries the status libr3d's
 * entry gives for the same defect and in the same precedence, and the row geometry follows the
 * same rules (rows = numel / n; `group` clamped to n; a rank-1 operand is one row; a rank-2 operand
 * whose width is not n is read flat):
 *   quant_act_fp8      src/r3d_band.hip:459-489     x, q, scale
 *   gated_quant_fp8    src/r3d_band.hip:491-548     gate_up, q, scale, out_bf16?
 *   rmsnorm_quant_fp8  src/r3d_more.hip:480-541     x, residual?, w, q, scale, out_bf16?
 * and the logits consumer of the column-sharded LM head:
 *   row_topk           src/r3d_more.hip:438-476     x, idx, val, pairs?
 *   sample_argmax      src/r3d_sample.hip:607-623   logits, params (not read), token
 */
#include <cuda_runtime.h>
#include "entry_util.h"
#include "r3d_kernels.h"

using namespace r3d;

namespace {

bool act_dtype(uint32_t dt) { return dt == RAD_F32 || dt == RAD_BF16; }

/* pitch (elements) of a row-major [rows, cols] operand; non-zero on a layout the kernels cannot walk */
int pitch_of(const RadTensor* t, int64_t cols, int64_t* pitch) {
    if (!t || !t->data) return 1;
    if (t->rank == 1) {
        if (rad_tensor_numel(t) != cols || t->stride[0] != 1) return 2;
        *pitch = 0;
        return 0;
    }
    if (t->rank < 1) return 2;
    const int last = (int)t->rank - 1;
    if (t->stride[last] != 1) return 3;
    if (t->rank == 2) {
        *pitch = t->shape[1] == cols ? t->stride[0] : cols;
        return 0;
    }
    if (t->shape[last] == cols)
        for (int i = 0; i < last; ++i)
            if (t->stride[i] != t->shape[i + 1] * t->stride[i + 1]) return 4;   /* a hole: not a flat walk */
    *pitch = cols;
    return 0;
}

int64_t int_param(const RadArgs* a, const char* key, int64_t fallback) {
    long long v;
    return rad_args_geti(a, key, &v) ? (int64_t)v : fallback;
}

const RadTensor* optional_out(const RadArgs* a, int i) {
    return (a->n_t > i && a->t[i].data) ? &a->t[i] : nullptr;
}

} /* namespace */

extern "C" int r3d_rad_quant_act_fp8(const RadArgs* a, RadStream s) {
    const RadTensor* x = rad_arg_in(a, 0);
    const RadTensor* q = rad_arg_in(a, 1);
    const RadTensor* sc = rad_arg_in(a, 2);
    if (!x || !q || !sc) return RAD_E_INVAL;
    if (!act_dtype(x->dtype)) return RAD_E_DTYPE;
    if (q->dtype != RAD_F8E4M3 || sc->dtype != RAD_F32) return RAD_E_DTYPE;
    const int64_t n = int_param(a, "n", x->rank >= 2 ? x->shape[1] : 0);
    if (n <= 0 || n > kMaxExtent) return RAD_E_SHAPE;
    const int64_t rows = rad_tensor_numel(x) / n;
    if (rows <= 0 || rows > 0xffff) return RAD_E_SHAPE;
    int64_t g = int_param(a, "group", n);
    if (g <= 0 || g > n) g = n;
    const int64_t ngrp = (n + g - 1) / g;
    if (rad_tensor_numel(q) < rows * n || rad_tensor_numel(sc) < rows * ngrp) return RAD_E_SHAPE;
    int64_t xp, qp, sp;
    if (pitch_of(x, n, &xp) || pitch_of(q, n, &qp) || pitch_of(sc, ngrp, &sp)) return RAD_E_STRIDE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_quant_act_fp8(x->data, (int)x->dtype, xp, q->data, qp, (float*)sc->data, sp, (int)rows, (int)n,
                                (int)g, (cudaStream_t)(uintptr_t)s);
}

extern "C" int r3d_rad_gated_quant_fp8(const RadArgs* a, RadStream s) {
    const RadTensor* gu = rad_arg_in(a, 0);
    const RadTensor* q = rad_arg_in(a, 1);
    const RadTensor* sc = rad_arg_in(a, 2);
    const RadTensor* ob = optional_out(a, 3);
    if (!gu || !q || !sc) return RAD_E_INVAL;
    if (!act_dtype(gu->dtype)) return RAD_E_DTYPE;
    if (q->dtype != RAD_F8E4M3 || sc->dtype != RAD_F32) return RAD_E_DTYPE;
    if (ob && !act_dtype(ob->dtype)) return RAD_E_DTYPE;
    const int64_t n = int_param(a, "n", gu->rank >= 2 ? gu->shape[1] / 2 : 0);
    if (n <= 0 || n > kMaxExtent / 2) return RAD_E_SHAPE;
    const char* act = rad_args_gets(a, "act");
    const int silu = !act || strcmp(act, "sigmoid") != 0;          /* absent or "silu": gate * sigmoid(gate) * up */
    int64_t g = int_param(a, "group", n);
    if (g <= 0 || g > n) g = n;
    const int64_t ngrp = (n + g - 1) / g;
    const int64_t rows = rad_tensor_numel(gu) / (2 * n);
    if (rows <= 0 || rows > 0xffff) return RAD_E_SHAPE;
    if (rad_tensor_numel(q) < rows * n || rad_tensor_numel(sc) < rows * ngrp) return RAD_E_SHAPE;
    if (ob && rad_tensor_numel(ob) < rows * n) return RAD_E_SHAPE;
    int64_t gp, qp, sp, op = 0;
    if (pitch_of(gu, 2 * n, &gp) || pitch_of(q, n, &qp) || pitch_of(sc, ngrp, &sp)) return RAD_E_STRIDE;
    if (ob && pitch_of(ob, n, &op)) return RAD_E_STRIDE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_gated_quant_fp8(gu->data, gp, q->data, qp, (float*)sc->data, sp, ob ? ob->data : nullptr,
                                  ob ? (int)ob->dtype : RAD_F32, op, (int)rows, (int)n, (int)g, silu,
                                  (cudaStream_t)(uintptr_t)s, (int)gu->dtype);
}

extern "C" int r3d_rad_rmsnorm_quant_fp8(const RadArgs* a, RadStream s) {
    if (a->n_t < 5) return RAD_E_INVAL;
    const RadTensor* x = rad_arg_in(a, 0);
    const RadTensor* res = optional_out(a, 1);
    const RadTensor* w = rad_arg_in(a, 2);
    const RadTensor* q = rad_arg_in(a, 3);
    const RadTensor* sc = rad_arg_in(a, 4);
    const RadTensor* ob = optional_out(a, 5);
    if (!x || !w || !q || !sc) return RAD_E_INVAL;
    if (x->dtype != RAD_BF16) return RAD_E_DTYPE;
    if (res && res->dtype != RAD_BF16) return RAD_E_DTYPE;         /* the sum narrows to the residual's dtype */
    if (!act_dtype(w->dtype)) return RAD_E_DTYPE;
    if (q->dtype != RAD_F8E4M3 || sc->dtype != RAD_F32) return RAD_E_DTYPE;
    if (ob && !act_dtype(ob->dtype)) return RAD_E_DTYPE;
    const int64_t n = int_param(a, "n", w->rank ? w->shape[w->rank - 1] : 0);
    if (n <= 0 || n > 30720) return RAD_E_SHAPE;                   /* the row is staged in shared memory */
    int64_t g = int_param(a, "group", 0);
    if (g <= 0 || g > n) g = n;
    const int64_t ngrp = (n + g - 1) / g;
    const float eps = (float)rad_args_getf_or(a, "eps", 1e-6);
    const float wadd = (float)rad_args_getf_or(a, "wadd", 0.0);
    const int64_t rows = rad_tensor_numel(x) / n;
    if (rows <= 0 || rows > 0xffff) return RAD_E_SHAPE;
    if (rad_tensor_numel(q) < rows * n || rad_tensor_numel(sc) < rows * ngrp || rad_tensor_numel(w) < n)
        return RAD_E_SHAPE;
    if (res && rad_tensor_numel(res) < rows * n) return RAD_E_SHAPE;
    if (ob && rad_tensor_numel(ob) < rows * n) return RAD_E_SHAPE;
    int64_t xp, rp = 0, qp, sp, op = 0;
    if (pitch_of(x, n, &xp)) return RAD_E_STRIDE;
    if (res && pitch_of(res, n, &rp)) return RAD_E_STRIDE;
    if (w->rank != 1 || w->stride[0] != 1) return RAD_E_STRIDE;
    if (pitch_of(q, n, &qp) || pitch_of(sc, ngrp, &sp)) return RAD_E_STRIDE;
    if (ob && pitch_of(ob, n, &op)) return RAD_E_STRIDE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_rmsnorm_quant_fp8(x->data, xp, res ? res->data : nullptr, rp, w->data, (int)w->dtype, q->data, qp,
                                    (float*)sc->data, sp, ob ? ob->data : nullptr, ob ? (int)ob->dtype : RAD_F32, op,
                                    (int)rows, (int)n, (int)g, eps, wadd, (cudaStream_t)(uintptr_t)s);
}

extern "C" int r3d_rad_row_topk(const RadArgs* a, RadStream s) {
    const RadTensor* x = rad_arg_in(a, 0);
    const RadTensor* idx = rad_arg_in(a, 1);
    const RadTensor* val = rad_arg_in(a, 2);
    const RadTensor* pairs = optional_out(a, 3);
    if (!x || !idx || !val) return RAD_E_INVAL;
    if (!act_dtype(x->dtype)) return RAD_E_DTYPE;
    if (idx->dtype != RAD_I32 || val->dtype != RAD_F32) return RAD_E_DTYPE;
    if (pairs && pairs->dtype != RAD_F32) return RAD_E_DTYPE;
    const int64_t N = int_param(a, "N", x->rank >= 2 ? x->shape[1] : 0);
    const int64_t R = int_param(a, "R", 1);
    const int64_t off = int_param(a, "vocab_off", 0);
    if (N <= 0 || N > kMaxExtent || R <= 0 || R > 32) return RAD_E_SHAPE;
    const int64_t M = rad_tensor_numel(x) / N;
    if (M <= 0 || M > 0xffff || rad_tensor_numel(idx) < M * R || rad_tensor_numel(val) < M * R) return RAD_E_SHAPE;
    if (pairs && rad_tensor_numel(pairs) < M * R * 2) return RAD_E_SHAPE;
    int64_t xp, ip, vp, pp = 0;
    if (pitch_of(x, N, &xp) || pitch_of(idx, R, &ip) || pitch_of(val, R, &vp)) return RAD_E_STRIDE;
    if (pairs) {
        /* [M, R, 2] as the schema describes it, or the same memory as a flat [M, 2R] */
        if (pairs->rank == 3) {
            if (pairs->stride[2] != 1 || pairs->stride[1] != 2 || pairs->stride[0] != 2 * R) return RAD_E_STRIDE;
            pp = 2 * R;
        } else if (pitch_of(pairs, 2 * R, &pp)) return RAD_E_STRIDE;
    }
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_row_topk(x->data, (int)x->dtype, xp, (int32_t*)idx->data, ip, (float*)val->data, vp,
                           pairs ? (float*)pairs->data : nullptr, pp, (int)M, (int)N, (int)R, off,
                           (cudaStream_t)(uintptr_t)s, a->scratch, a->scratch_bytes);
}

/* the launch arena of row_topk: the tournament's two survivor planes (src/r3d_more.hip's row needs none: it
 * re-reads the row R times from one block instead). With the arena the row allocates nothing; without one
 * it falls back to planes of its own, allocated on first use. */
extern "C" int64_t r3d_rad_row_topk_scratch(const RadArgs* a) {
    const RadTensor* x = rad_arg_in(a, 0);
    const int64_t N = int_param(a, "N", x && x->rank >= 2 ? x->shape[1] : 0);
    const int64_t R = int_param(a, "R", 1);
    if (N <= 0 || N > kMaxExtent || R <= 0 || R > 32) return 0;
    /* M from the operand when it is there, else the query's M (an upper bound is what an arena wants) */
    const int64_t M = x ? rad_tensor_numel(x) / N : int_param(a, "M", 0);
    return M > 0 && M <= 0xffff ? r3d::row_topk_scratch_bytes(M, N, R) : 0;
}

/* Greedy sampling: token[m] = the column of the row's largest logit, ties to the lower token id --
 * the top-1 of the same total order, so it is the same tournament with R = 1. The per-row parameter
 * blob (operand 1) is not read, as in the reference. */
extern "C" int r3d_rad_sample_argmax(const RadArgs* a, RadStream s) {
    const RadTensor* lg = rad_arg_in(a, 0);
    const RadTensor* tok = rad_arg_in(a, 2);
    if (!lg || !tok) return RAD_E_INVAL;
    if (lg->dtype != RAD_F32 || tok->dtype != RAD_I32) return RAD_E_DTYPE;
    long long nv = 0;
    if (!rad_args_geti(a, "n_vocab", &nv) || nv <= 0) nv = lg->rank >= 2 ? lg->shape[1] : 0;
    if (nv <= 0 || nv > kMaxExtent) return RAD_E_SHAPE;
    const int64_t M = rad_tensor_numel(lg) / nv;
    if (M <= 0 || M > 0xffff) return RAD_E_SHAPE;
    if (rad_tensor_numel(tok) < M || tok->rank != 1 || tok->stride[0] != 1) return RAD_E_SHAPE;
    if (lg->rank != 2 || lg->shape[1] != nv || lg->stride[1] != 1) return RAD_E_STRIDE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_row_topk(lg->data, RAD_F32, lg->stride[0], (int32_t*)tok->data, 1, nullptr, 0, nullptr, 0, (int)M,
                           (int)nv, 1, 0, (cudaStream_t)(uintptr_t)s, a->scratch, a->scratch_bytes);
}

extern "C" int64_t r3d_rad_sample_argmax_scratch(const RadArgs* a) {
    const RadTensor* lg = rad_arg_in(a, 0);
    long long nv = 0;
    if (!rad_args_geti(a, "n_vocab", &nv) || nv <= 0) nv = lg && lg->rank >= 2 ? lg->shape[1] : 0;
    if (nv <= 0 || nv > kMaxExtent) return 0;
    const int64_t M = lg ? rad_tensor_numel(lg) / nv : int_param(a, "M", 0);
    return M > 0 && M <= 0xffff ? r3d::row_topk_scratch_bytes(M, nv, 1) : 0;
}

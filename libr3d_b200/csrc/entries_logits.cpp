/* entries_logits.cpp -- the logits_gemm row over a joined e4m3 + block-scale LM head, and
 * the row's three layout hooks. Host C++ only.
 *
 * Mirrors src/r3d_gemm_logits.hip:145-272: operands (x, lm_head, logits); dtype "bf16";
 * x bf16, logits f32; M = numel(logits) / n_vocab; the head is a rad.planes blob holding
 * exactly a `codes` plane (e4m3, block 1x1, dense rows) and a `scale` plane (bf16, f16 or
 * f32, one element per (1 or 128 rows, 128 columns)), untransformed.
 *
 * One difference forced by the platform: the reference reads the blob header through the
 * operand pointer on the host, which works where device memory is host-visible. A CUDA
 * device allocation is not, so the header and entries of a device-resident blob are copied
 * to the host once, on first sight of that pointer, and remembered (weights are immortal
 * for the life of the engine). That first call synchronises; later calls do not.
 */
#include <cstdio>
#include <vector>
#include <cuda_runtime.h>
#include "entry_util.h"
#include "rad_planes.h"
#include "r3d_b200.h"
#include "r3d_kernels.h"

using namespace r3d;

namespace {

struct HeadPlanes { const RadPlanesHeader* h; const RadPlanesEntry* ec; const RadPlanesEntry* es; };

/* the checks of src/r3d_gemm_logits.hip:176-194 of libr3d on a host copy of the header */
int check_head(const unsigned char* hv, long long N, long long K, HeadPlanes* out, int not_joined) {
    const RadPlanesHeader* h = hv ? rad_planes_header(hv) : nullptr;
    if (!h || h->n_planes != 2) return h ? RAD_E_DTYPE : not_joined;
    if (h->transform[0]) return RAD_E_UNSUPPORTED;
    const RadPlanesEntry* ec = nullptr;
    const RadPlanesEntry* es = nullptr;
    if (!rad_planes_find(hv, "codes", &ec) || !rad_planes_find(hv, "scale", &es) || !ec || !es)
        return RAD_E_DTYPE;
    if (ec->dtype != RAD_F8E4M3 || ec->block[0] != 1 || ec->block[1] != 1 ||
        ec->rows != N || ec->cols != K) return RAD_E_SHAPE;
    out->h = h; out->ec = ec; out->es = es;
    return RAD_OK;
}

} /* namespace */

extern "C" {

int r3d_rad_logits_gemm_e4m3(const RadArgs* a, RadStream s) {
    const RadTensor* X = rad_arg_in(a, 0);
    const RadTensor* W = rad_arg_in(a, 1);
    const RadTensor* Y = rad_arg_in(a, 2);
    if (!X || !W || !Y) return RAD_E_UNSUPPORTED;
    const char* dt = rad_args_gets(a, "dtype");
    if (!dt || strcmp(dt, "bf16") != 0) return RAD_E_UNSUPPORTED;
    if (X->dtype != RAD_BF16 || Y->dtype != RAD_F32) return RAD_E_UNSUPPORTED;

    long long N = 0, K = 0;
    if (!rad_args_geti(a, "n_vocab", &N) || !rad_args_geti(a, "n_embd", &K)) return RAD_E_SHAPE;
    if (N <= 0 || K <= 0) return RAD_E_SHAPE;
    const long long Yn = rad_tensor_numel(Y);
    if (Yn <= 0 || Yn % N) return RAD_E_SHAPE;
    const long long M = Yn / N;
    if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return RAD_E_SHAPE;
    if (rad_tensor_numel(X) < M * K) return RAD_E_SHAPE;
    if ((K & 3) != 0) return RAD_E_UNSUPPORTED;

    if (!inner_contiguous(X) || !inner_contiguous(Y)) return RAD_E_STRIDE;
    const int64_t x_pitch = X->rank >= 2 ? X->stride[X->rank - 2] : K;
    const int64_t y_pitch = Y->rank >= 2 ? Y->stride[Y->rank - 2] : N;
    if (x_pitch < K || y_pitch < N) return RAD_E_STRIDE;

    bool cached = false;
    const unsigned char* hv = planes_head_of(W->data, &cached);
    HeadPlanes hp{};
    int hst = check_head(hv, N, K, &hp, RAD_E_DTYPE);
    if (hst != RAD_OK && cached) hst = check_head(planes_head_refresh(W->data), N, K, &hp, RAD_E_DTYPE);
    if (hst != RAD_OK) return hst;
    const RadPlanesHeader* h = hp.h;
    const RadPlanesEntry* ec = hp.ec;
    const RadPlanesEntry* es = hp.es;
    if (es->dtype != RAD_BF16 && es->dtype != RAD_F16 && es->dtype != RAD_F32)
        return RAD_E_UNSUPPORTED;
    if (es->block[1] != 128 || (es->block[0] != 1 && es->block[0] != 128)) return RAD_E_UNSUPPORTED;
    const int64_t srows = (N + es->block[0] - 1) / es->block[0];
    const int64_t scols = (K + 127) / 128;
    if (es->rows != srows || es->cols != scols) return RAD_E_SHAPE;
    if (ec->row_bytes != K) return RAD_E_STRIDE;
    if ((int64_t)h->bytes < es->offset + es->rows * es->row_bytes) return RAD_E_SHAPE;

    R3dLogits l{};
    l.x = X->data;
    l.codes = (const unsigned char*)W->data + ec->offset;
    l.scale = (const unsigned char*)W->data + es->offset;
    l.y = Y->data;
    l.m = (int32_t)M; l.n = (int32_t)N; l.k = (int32_t)K;
    l.br = (int32_t)es->block[0];
    l.scale_dtype = (int32_t)es->dtype;
    l.y_dtype = RAD_F32;
    l.head_fmt = 0;
    l.arm = R3D_ARM_AUTO;
    l.x_pitch = x_pitch; l.code_pitch = ec->row_bytes; l.y_pitch = y_pitch;
    l.scale_pitch = es->row_bytes / (es->dtype == RAD_F32 ? 4 : 2);
    return r3d_b200_logits(&l, (void*)s);
}

/* logit_rerank over the joined e4m3 head (src/r3d_logit_rerank_e4m3.hip:226-345 of libr3d): operands
 * x, head, idx_in, idx, val, pairs?; R <= 32; M = numel(x) / n_embd, never the M parameter; the same
 * refusal order and codes as the reference's entry. */
int r3d_rad_logit_rerank_e4m3(const RadArgs* a, RadStream s) {
    static const bool off = env_present("R3D_NO_DFLASH");
    if (off) return RAD_E_UNSUPPORTED;
    if (a->n_t < 5) return RAD_E_INVAL;
    const RadTensor* x = rad_arg_in(a, 0);
    const RadTensor* w = rad_arg_in(a, 1);
    const RadTensor* in = rad_arg_in(a, 2);
    const RadTensor* idx = rad_arg_in(a, 3);
    const RadTensor* val = rad_arg_in(a, 4);
    const RadTensor* pairs = (a->n_t > 5 && a->t[5].data) ? &a->t[5] : nullptr;
    if (!x || !w || !in || !idx || !val) return RAD_E_INVAL;
    long long R = 1, K = 0, NV = 0, voff = 0, v = 0;
    if (rad_args_geti(a, "R", &v)) R = v;
    if (rad_args_geti(a, "n_embd", &v)) K = v;
    if (rad_args_geti(a, "n_vocab", &v)) NV = v;
    if (rad_args_geti(a, "vocab_off", &v)) voff = v;
    if (R <= 0 || K <= 0 || NV <= 0) return RAD_E_SHAPE;
    if (R > 32) return RAD_E_UNSUPPORTED;
    const long long M = rad_tensor_numel(x) / K;
    if (M <= 0 || M > 0xffff) return RAD_E_SHAPE;
    if (rad_tensor_numel(in) < M * R || rad_tensor_numel(idx) < M * R || rad_tensor_numel(val) < M * R)
        return RAD_E_SHAPE;
    if (x->dtype != RAD_F32 && x->dtype != RAD_BF16) return RAD_E_DTYPE;
    if (in->dtype != RAD_I32 || idx->dtype != RAD_I32 || val->dtype != RAD_F32) return RAD_E_DTYPE;

    bool cached = false;
    const unsigned char* hv = planes_head_of(w->data, &cached);
    HeadPlanes hp{};
    int hst = check_head(hv, NV, K, &hp, RAD_E_UNSUPPORTED);
    if (hst != RAD_OK && cached) hst = check_head(planes_head_refresh(w->data), NV, K, &hp, RAD_E_UNSUPPORTED);
    if (hst != RAD_OK) return hst;
    const RadPlanesEntry* ec = hp.ec;
    const RadPlanesEntry* es = hp.es;
    if (ec->row_bytes != K) return RAD_E_STRIDE;
    if (es->dtype != RAD_BF16 && es->dtype != RAD_F16 && es->dtype != RAD_F32) return RAD_E_DTYPE;
    if (es->block[1] != 128 || (es->block[0] != 1 && es->block[0] != 128)) return RAD_E_DTYPE;
    const int64_t srows = (NV + es->block[0] - 1) / es->block[0];
    const int64_t scols = (K + 127) / 128;
    if (es->rows != srows || es->cols != scols) return RAD_E_SHAPE;
    if ((int64_t)hp.h->bytes < es->offset + es->rows * es->row_bytes) return RAD_E_SHAPE;
    const int64_t sbytes = es->dtype == RAD_F32 ? 4 : 2;
    if (es->row_bytes < scols * sbytes) return RAD_E_STRIDE;
    const int64_t scale_rs = es->row_bytes / sbytes;

    if (pairs && (pairs->dtype != RAD_F32 || rad_tensor_numel(pairs) < M * R * 2)) return RAD_E_SHAPE;
    if (pairs) {
        if (pairs->rank == 3) {
            if (pairs->stride[2] != 1 || pairs->stride[1] != 2 || pairs->stride[0] != 2 * R) return RAD_E_STRIDE;
        } else if (pairs->rank != 2 || pairs->stride[1] != 1 || pairs->stride[0] < 2 * R) return RAD_E_STRIDE;
    }
    auto row2 = [](const RadTensor* t, int64_t cols, int64_t* pitch) {
        if (!t || t->rank != 2 || t->stride[1] != 1) return false;
        *pitch = (t->shape[1] == cols) ? t->stride[0] : cols;
        return true;
    };
    int64_t xp = 0, ip = 0, op = 0, vp = 0;
    if (!row2(x, K, &xp) || !row2(in, R, &ip) || !row2(idx, R, &op) || !row2(val, R, &vp)) return RAD_E_STRIDE;
    if (!r3d::device_is_sm100()) return RAD_E_UNSUPPORTED;
    return r3d::launch_logit_rerank_e4m3(x->data, (int)x->dtype, xp, (const unsigned char*)w->data + ec->offset,
                                         ec->row_bytes, (const unsigned char*)w->data + es->offset, scale_rs,
                                         (int)es->block[0], (int)es->dtype, (const int32_t*)in->data, ip,
                                         (int32_t*)idx->data, op, (float*)val->data, vp,
                                         pairs ? (float*)pairs->data : nullptr, (int)M, (int)R, (int)K, NV, voff,
                                         (cudaStream_t)(uintptr_t)s);
}

/* Admit exactly "codes, then one scale", affine, untransformed -- and only e4m3 codes.
 * An int8 head is refused here so it resolves elsewhere at declare time, never at issue. */
int r3d_layout_head(const RadParam*, int, int operand, const RadEncoding* enc, const int* sel,
                    const RadTensor* planes, int n, RadLayout* out) {
    if (n < 2 || operand != 1) return RAD_E_UNSUPPORTED;
    if (!enc || !sel || n != 2) return RAD_E_UNSUPPORTED;
    for (int i = 0; i < 2; ++i)
        if (sel[i] < 0 || sel[i] >= enc->n_planes) return RAD_E_DTYPE;
    if (enc->n_planes != 2 || enc->transform[0]) return RAD_E_DTYPE;
    if (strncmp(enc->plane[sel[0]].role, "codes", RAD_ENC_STR) != 0 ||
        strncmp(enc->plane[sel[1]].role, "scale", RAD_ENC_STR) != 0) return RAD_E_DTYPE;
    const RadEncPlane& c = enc->plane[sel[0]];
    const RadEncPlane& sc = enc->plane[sel[1]];
    if (c.kind != RAD_PLANE_TILED || c.block[0] != 1 || c.block[1] != 1 || c.dtype != RAD_F8E4M3)
        return RAD_E_DTYPE;
    if (sc.kind != RAD_PLANE_TILED ||
        (sc.dtype != RAD_BF16 && sc.dtype != RAD_F16 && sc.dtype != RAD_F32)) return RAD_E_DTYPE;
    if (strncmp(enc->scheme, "affine", RAD_ENC_STR) != 0) return RAD_E_DTYPE;
    return rad_planes_layout(enc, sel, planes, n, out);
}

int r3d_relayout_head(const RadParam* p, int n_p, int operand, const RadEncoding* enc,
                      const int* sel, const RadTensor* planes, int n, void* dst,
                      int64_t dst_bytes) {
    RadLayout lay;
    const int st = r3d_layout_head(p, n_p, operand, enc, sel, planes, n, &lay);
    if (st != RAD_OK) return st;
    return rad_planes_relayout(enc, sel, planes, n, dst, dst_bytes);
}

int r3d_unrelayout_head(const RadParam* p, int n_p, int operand, const RadEncoding* enc,
                        const int* sel, const void* src, int64_t src_bytes,
                        const RadTensor* planes, int n) {
    RadLayout lay;
    const int st = r3d_layout_head(p, n_p, operand, enc, sel, planes, n, &lay);
    if (st != RAD_OK) return st;
    return rad_planes_unrelayout(enc, sel, src, src_bytes, planes, n);
}

} /* extern "C" */

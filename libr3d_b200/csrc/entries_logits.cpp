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

using namespace r3d;

namespace {

struct HeadView {
    const void* blob;               /* key: the operand's data pointer */
    alignas(16) unsigned char head[sizeof(RadPlanesHeader) +
                                   RAD_ENC_MAX_PLANES * sizeof(RadPlanesEntry)];
};

/* Host-readable copy of the blob's header + entry table, or nullptr. */
const unsigned char* head_of(const void* blob) {
    static std::vector<HeadView*> seen;
    for (const HeadView* v : seen) if (v->blob == blob) return v->head;
    cudaPointerAttributes at{};
    const bool have = cudaPointerGetAttributes(&at, blob) == cudaSuccess;
    if (!have) (void)cudaGetLastError();
    HeadView* v = new HeadView;
    v->blob = blob;
    if (have && at.type == cudaMemoryTypeDevice) {
        if (cudaMemcpy(v->head, blob, sizeof v->head, cudaMemcpyDeviceToHost) != cudaSuccess) {
            (void)cudaGetLastError();
            delete v;
            return nullptr;
        }
    } else {
        memcpy(v->head, blob, sizeof v->head);      /* host, pinned or managed memory */
    }
    seen.push_back(v);
    return v->head;
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

    const unsigned char* hv = head_of(W->data);
    const RadPlanesHeader* h = hv ? rad_planes_header(hv) : nullptr;
    if (!h || h->n_planes != 2) return RAD_E_DTYPE;
    if (h->transform[0]) return RAD_E_UNSUPPORTED;
    const RadPlanesEntry* ec = nullptr;
    const RadPlanesEntry* es = nullptr;
    if (!rad_planes_find(hv, "codes", &ec) || !rad_planes_find(hv, "scale", &es) || !ec || !es)
        return RAD_E_DTYPE;
    if (ec->dtype != RAD_F8E4M3 || ec->block[0] != 1 || ec->block[1] != 1 ||
        ec->rows != N || ec->cols != K) return RAD_E_SHAPE;
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

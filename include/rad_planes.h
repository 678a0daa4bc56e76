/* rad_planes.h -- clean-room stand-in for radiance's joined-weight blob ("rad.planes").
 *
 * A joined weight is one allocation: a header, `n_planes` entries, then each plane's
 * payload at its entry's `offset`. libr3d's LM-head row receives its operand 1 in this
 * form (src/r3d_gemm_logits.hip:176-194) and its layout hooks delegate to these helpers
 * (src/r3d_gemm_logits.hip:233-272). Field names and the construction recipe follow the
 * reference's own blob builder, tools/bench_w2a8.cpp:84-105. The magic spells "PLNS"
 * (docs/COVERAGE.md:1163). UNPINNED (real header absent): exact packing, the rounding
 * granule of rad_planes_round, the tag string. All three live only in this file.
 *
 * Host-side helpers only: every function here dereferences the blob on the host.
 */
#ifndef RAD_PLANES_H
#define RAD_PLANES_H

#include "rad_abi.h"
#include "rad_plugin.h"
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RAD_PLANES_MAGIC 0x534E4C50u   /* 'P','L','N','S' little-endian */
#define RAD_PLANES_ALIGN 256           /* UNPINNED granule */

typedef struct RadPlanesHeader {
    uint32_t magic;
    uint32_t n_planes;
    char     transform[RAD_ENC_STR];
    int64_t  bytes;          /* whole blob, header included */
} RadPlanesHeader;

typedef struct RadPlanesEntry {
    char     role[RAD_ENC_STR];
    uint32_t dtype;
    int32_t  kind;
    int64_t  block[2];       /* rows x cols of the weight one element of this plane covers */
    int64_t  rows, cols;     /* extent of the plane itself */
    int64_t  row_bytes;
    int64_t  offset;         /* payload, from the blob's first byte */
} RadPlanesEntry;

static inline int64_t rad_planes_round(int64_t x) {
    return (x + (RAD_PLANES_ALIGN - 1)) / RAD_PLANES_ALIGN * RAD_PLANES_ALIGN;
}

static inline const RadPlanesHeader* rad_planes_header(const void* blob) {
    const RadPlanesHeader* h = (const RadPlanesHeader*)blob;
    if (!h || h->magic != RAD_PLANES_MAGIC) return NULL;
    if (h->n_planes == 0 || h->n_planes > RAD_ENC_MAX_PLANES) return NULL;
    return h;
}

static inline const RadPlanesEntry* rad_planes_entries(const void* blob) {
    return (const RadPlanesEntry*)((const char*)blob + sizeof(RadPlanesHeader));
}

/* Payload pointer of the plane whose role is `role`, or NULL. */
static inline const void* rad_planes_find(const void* blob, const char* role,
                                          const RadPlanesEntry** entry) {
    const RadPlanesHeader* h = rad_planes_header(blob);
    if (!h) return NULL;
    const RadPlanesEntry* e = rad_planes_entries(blob);
    for (uint32_t i = 0; i < h->n_planes; ++i)
        if (strncmp(e[i].role, role, RAD_ENC_STR) == 0) {
            if (entry) *entry = &e[i];
            return (const char*)blob + e[i].offset;
        }
    return NULL;
}

/* Size and tag of the blob that joins the selected planes, in selection order. */
static inline int rad_planes_layout(const RadEncoding* enc, const int* sel,
                                    const RadTensor* planes, int n, RadLayout* out) {
    if (!enc || !sel || !planes || !out || n < 1 || n > RAD_ENC_MAX_PLANES) return RAD_E_INVAL;
    int64_t off = rad_planes_round((int64_t)(sizeof(RadPlanesHeader) +
                                             (size_t)n * sizeof(RadPlanesEntry)));
    for (int i = 0; i < n; ++i) {
        if (planes[i].rank < 2) return RAD_E_SHAPE;
        const int64_t rb = rad_dtype_bytes(planes[i].dtype, planes[i].shape[1]);
        off = rad_planes_round(off + planes[i].shape[0] * rb);
    }
    out->bytes = off;
    out->align = RAD_PLANES_ALIGN;
    out->tag   = "rad.planes";
    return RAD_OK;
}

static inline int rad_planes_relayout(const RadEncoding* enc, const int* sel,
                                      const RadTensor* planes, int n, void* dst,
                                      int64_t dst_bytes) {
    RadLayout lay;
    int st = rad_planes_layout(enc, sel, planes, n, &lay);
    if (st != RAD_OK) return st;
    if (!dst || dst_bytes < lay.bytes) return RAD_E_SHAPE;
    RadPlanesHeader* h = (RadPlanesHeader*)dst;
    memset(dst, 0, (size_t)rad_planes_round((int64_t)(sizeof(RadPlanesHeader) +
                                                      (size_t)n * sizeof(RadPlanesEntry))));
    h->magic = RAD_PLANES_MAGIC;
    h->n_planes = (uint32_t)n;
    memcpy(h->transform, enc->transform, RAD_ENC_STR);
    h->bytes = lay.bytes;
    RadPlanesEntry* e = (RadPlanesEntry*)((char*)dst + sizeof(RadPlanesHeader));
    int64_t off = rad_planes_round((int64_t)(sizeof(RadPlanesHeader) +
                                             (size_t)n * sizeof(RadPlanesEntry)));
    for (int i = 0; i < n; ++i) {
        const RadEncPlane* ep = &enc->plane[sel[i]];
        const int64_t rb = rad_dtype_bytes(planes[i].dtype, planes[i].shape[1]);
        memcpy(e[i].role, ep->role, RAD_ENC_STR);
        e[i].dtype = planes[i].dtype;
        e[i].kind = ep->kind;
        e[i].block[0] = ep->block[0]; e[i].block[1] = ep->block[1];
        e[i].rows = planes[i].shape[0]; e[i].cols = planes[i].shape[1];
        e[i].row_bytes = rb;
        e[i].offset = off;
        if (!planes[i].data) return RAD_E_INVAL;
        const int64_t src_pitch = rad_dtype_bytes(planes[i].dtype, planes[i].stride[0]);
        for (int64_t r = 0; r < e[i].rows; ++r)
            memcpy((char*)dst + off + r * rb, (const char*)planes[i].data + r * src_pitch,
                   (size_t)rb);
        off = rad_planes_round(off + e[i].rows * rb);
    }
    return RAD_OK;
}

static inline int rad_planes_unrelayout(const RadEncoding* enc, const int* sel,
                                        const void* src, int64_t src_bytes,
                                        const RadTensor* planes, int n) {
    (void)enc; (void)sel;
    const RadPlanesHeader* h = rad_planes_header(src);
    if (!h || (int)h->n_planes != n || src_bytes < h->bytes) return RAD_E_SHAPE;
    const RadPlanesEntry* e = rad_planes_entries(src);
    for (int i = 0; i < n; ++i) {
        if (!planes[i].data || planes[i].rank < 2) return RAD_E_INVAL;
        if (planes[i].shape[0] != e[i].rows || planes[i].shape[1] != e[i].cols)
            return RAD_E_SHAPE;
        const int64_t dst_pitch = rad_dtype_bytes(planes[i].dtype, planes[i].stride[0]);
        for (int64_t r = 0; r < e[i].rows; ++r)
            memcpy((char*)planes[i].data + r * dst_pitch,
                   (const char*)src + e[i].offset + r * e[i].row_bytes, (size_t)e[i].row_bytes);
    }
    return RAD_OK;
}

#ifdef __cplusplus
}
#endif
#endif /* RAD_PLANES_H */

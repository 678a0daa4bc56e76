/* rad_plugin.h -- clean-room stand-in for the host-side helpers a radiance kernel plugin
 * uses to read its RadArgs. Reconstructed from call sites in libr3d:
 *   rad_arg_in        src/r3d_gemm_fp8a8.hip:1061-1067 (null when absent or data-less)
 *   rad_args_geti     src/r3d_gemm_fp8a8.hip:857-858   (bool, writes long long)
 *   rad_args_gets     src/r3d_gemm_fp8a8.hip:853
 *   rad_args_getf_or  src/r3d_kvstore.hip:312
 *   rad_tensor_numel  src/r3d_gemm_fp8a8.hip:871
 *   rad_dtype_bytes   src/r3d_logit_rerank_e4m3.hip:287
 * Header-only (static inline) so the plugin needs no engine library at link time.
 */
#ifndef RAD_PLUGIN_H
#define RAD_PLUGIN_H

#include "rad_abi.h"
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Operand `i` by schema position, or NULL when the caller passed fewer tensors or a
 * tensor without storage (how optional operands are spelled absent). */
static inline const RadTensor* rad_arg_in(const RadArgs* a, int i) {
    if (!a || !a->t || i < 0 || i >= a->n_t) return NULL;
    return a->t[i].data ? &a->t[i] : NULL;
}

static inline const RadParam* rad_args_find(const RadArgs* a, const char* key) {
    if (!a || !a->p || !key) return NULL;
    for (int i = 0; i < a->n_p; ++i)
        if (a->p[i].key && strcmp(a->p[i].key, key) == 0) return &a->p[i];
    return NULL;
}

static inline int rad_args_geti(const RadArgs* a, const char* key, long long* out) {
    const RadParam* p = rad_args_find(a, key);
    if (!p || p->kind != RAD_PK_INT) return 0;
    if (out) *out = p->ival;
    return 1;
}

static inline long long rad_args_geti_or(const RadArgs* a, const char* key, long long dflt) {
    long long v = dflt;
    return rad_args_geti(a, key, &v) ? v : dflt;
}

static inline const char* rad_args_gets(const RadArgs* a, const char* key) {
    const RadParam* p = rad_args_find(a, key);
    return (p && p->kind == RAD_PK_STR) ? p->sval : NULL;
}

static inline double rad_args_getf_or(const RadArgs* a, const char* key, double dflt) {
    const RadParam* p = rad_args_find(a, key);
    if (!p) return dflt;
    if (p->kind == RAD_PK_F64) return p->dval;
    if (p->kind == RAD_PK_INT) return (double)p->ival;
    return dflt;
}

static inline int64_t rad_tensor_numel(const RadTensor* t) {
    if (!t) return 0;
    int64_t n = 1;
    for (uint32_t i = 0; i < t->rank && i < RAD_MAX_RANK; ++i) n *= t->shape[i];
    return n;
}

/* Storage bytes of `n` elements of `dt` (sub-byte types round up to whole bytes). */
static inline int64_t rad_dtype_bytes(uint32_t dt, int64_t n) {
    switch (dt) {
        case RAD_F64: case RAD_I64:                return n * 8;
        case RAD_F32: case RAD_I32:                return n * 4;
        case RAD_F16: case RAD_BF16:               return n * 2;
        case RAD_F8E4M3: case RAD_F8E5M2:
        case RAD_E8M0: case RAD_U8: case RAD_I8:   return n;
        case RAD_FP4E2M1: case RAD_U4:             return (n + 1) / 2;
        case RAD_U2:                               return (n + 3) / 4;
        default:                                   return 0;
    }
}

#ifdef __cplusplus
}
#endif
#endif /* RAD_PLUGIN_H */

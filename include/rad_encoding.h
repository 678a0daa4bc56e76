/* rad_encoding.h -- clean-room stand-in for radiance's header of that name, reconstructed from the one
 * place libr3d uses it: src/r3d_gemm_w2a8.hip:112 includes it and calls rad_param_geti(p, n_p, key,
 * fallback) in its layout hook (:1383-1391) to read declare-time parameters from a bare RadParam
 * array (the hooks get no RadArgs). The encoding types themselves (RadEncoding, RadEncPlane) are
 * declared by rad_abi.h in this stand-in set. Header-only. */
#ifndef RAD_ENCODING_H
#define RAD_ENCODING_H

#include "rad_abi.h"
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

/* integer parameter `key` of a RadParam array, or `dflt` when absent or not an integer */
static inline long long rad_param_geti(const RadParam* p, int n_p, const char* key, long long dflt) {
    if (!p || !key) return dflt;
    for (int i = 0; i < n_p; ++i)
        if (p[i].key && strcmp(p[i].key, key) == 0) return p[i].kind == RAD_PK_INT ? p[i].ival : dflt;
    return dflt;
}

#ifdef __cplusplus
}
#endif
#endif /* RAD_ENCODING_H */

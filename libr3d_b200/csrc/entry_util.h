/* entry_util.h -- shape arithmetic the row entries share. Host only. */
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include "rad_abi.h"
#include "rad_plugin.h"

namespace r3d {

/* Block size implied by a scale grid of `blocks` columns over an extent `ext`: the whole
 * extent for a single block; otherwise the smallest power of two >= ceil(ext/blocks) when
 * that power of two reproduces `blocks`, else ceil(ext/blocks). This is how the reference
 * derives a grid from tensor shapes instead of trusting the `group` parameter
 * (src/r3d_gemm_fp8a8.hip:58-67, src/r3d_gemm_mxfp4.hip:71-82). */
inline int64_t grid_block(int64_t ext, int64_t blocks) {
    if (ext <= 0) return 1;
    if (blocks <= 1) return ext;
    const int64_t need = (ext + blocks - 1) / blocks;
    int64_t pow2 = 1;
    while (pow2 < need) pow2 <<= 1;
    return ((ext + pow2 - 1) / pow2 == blocks) ? pow2 : need;
}

/* Row pitch (elements) of a tensor whose rows are `cols` wide: trailing dimensions are
 * folded until their product is `cols`; the stride of the next dimension out is the pitch
 * (rank-3 views are legal). src/r3d_gemm_fp8a8.hip:69-80. */
inline int64_t row_pitch(const RadTensor* t, int64_t cols) {
    if (!t || t->rank < 2) return cols;
    int64_t span = 1;
    for (int i = (int)t->rank - 1; i >= 0; --i) {
        span *= t->shape[i];
        if (span == cols) return i > 0 ? t->stride[i - 1] : cols;
        if (span > cols) break;
    }
    return t->stride[t->rank - 2];
}

inline bool inner_contiguous(const RadTensor* t) {
    return !(t->rank >= 2 && t->stride[t->rank - 1] != 1);
}

/* An environment lever that is ON when the variable exists, whatever its value. */
inline bool env_present(const char* name) { return getenv(name) != nullptr; }
/* A lever whose only OFF spelling is the literal "0" (README.md:106-127 of the reference). */
inline bool env_is_zero(const char* name) {
    const char* e = getenv(name);
    return e && !strcmp(e, "0");
}

/* Host-readable copy of a rad.planes blob's header + entry table (planes_cache.cpp), or nullptr.
 * `*cached` says whether the copy was taken by an earlier call; planes_head_refresh re-reads it. */
const unsigned char* planes_head_of(const void* blob, bool* cached);
const unsigned char* planes_head_refresh(const void* blob);

constexpr long long kMaxExtent = 0x7ffffffLL;   /* extents must fit the kernels' int math */

} /* namespace r3d */

/* rocwmma/rocwmma.hpp stand-in for the reference pin builds: rocWMMA's fragment API is the
 * nvcuda::wmma API under another namespace, so the reference's 16x16x16 bf16 tiles compile to
 * NVIDIA's warp-level MMA. rocWMMA also accepts a run-time layout on operand loads (the fragment
 * type already fixes it); that form forwards to the three-argument load. TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <mma.h>
#include <cuda_bf16.h>
namespace rocwmma {
using namespace nvcuda::wmma;
using bfloat16_t = __nv_bfloat16;
using nvcuda::wmma::load_matrix_sync;
template <int M, int N, int K, typename T, typename L>
__device__ inline void load_matrix_sync(fragment<matrix_a, M, N, K, T, L>& f, const T* p, unsigned ldm, layout_t) {
    nvcuda::wmma::load_matrix_sync(f, p, ldm);
}
template <int M, int N, int K, typename T, typename L>
__device__ inline void load_matrix_sync(fragment<matrix_b, M, N, K, T, L>& f, const T* p, unsigned ldm, layout_t) {
    nvcuda::wmma::load_matrix_sync(f, p, ldm);
}
}

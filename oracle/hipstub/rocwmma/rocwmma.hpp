/* rocwmma/rocwmma.hpp stand-in for the reference pin builds: rocWMMA's fragment API is the
 * nvcuda::wmma API under another namespace, so the reference's 16x16x16 bf16 tiles compile to
 * NVIDIA's warp-level MMA. TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <mma.h>
#include <cuda_bf16.h>
namespace rocwmma {
using namespace nvcuda::wmma;
using bfloat16_t = __nv_bfloat16;
}

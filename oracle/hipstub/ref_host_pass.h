/* ref_host_pass.h -- for a pin build that also wants the reference's pure __device__ helpers on the
 * CPU (they are compiled __host__ __device__ there): in the host compilation pass the device-only
 * intrinsics those files use get host meanings. Include after every CUDA header.
 * TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <cstdint>
#include <cstring>
#ifndef __CUDA_ARCH__
/* host pass: the reference's __device__ helpers are compiled __host__ __device__ (ref_band.cu) */
static inline float ref_host_u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t ref_host_f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
struct RefHostDim { unsigned x, y, z; };
static const RefHostDim ref_host_idx = {0, 0, 0};
#define __uint_as_float(u) ref_host_u2f(u)
#define __float_as_uint(f) ref_host_f2u(f)
#define __shfl_down_sync(m, v, o) (v)
#define __shfl_xor_sync(m, v, o) (v)
#define __syncthreads() ((void)0)
#define threadIdx ref_host_idx
#define blockIdx ref_host_idx
#endif

/* hip/hip_runtime.h -- a stand-in that lets nvcc compile libr3d's HIP sources where they lie,
 * for the reference pin only (oracle/ref_band.cu). It maps the handful of HIP runtime names those
 * files use onto CUDA's and, in the host compilation pass, gives the device-only intrinsics host
 * meanings so that the reference's pure __device__ helpers can also be called on the CPU.
 * TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>

typedef cudaStream_t hipStream_t;
typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
#define hipGetLastError cudaGetLastError
#define hipStreamSynchronize cudaStreamSynchronize

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

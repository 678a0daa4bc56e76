/* hip/hip_runtime.h -- a stand-in that lets nvcc compile libr3d's HIP sources where they lie,
 * for the reference pin only (oracle/ref_band.cu). It maps the handful of HIP runtime names those
 * files use onto CUDA's.
 * TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstring>

typedef cudaStream_t hipStream_t;
typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
#define hipGetLastError cudaGetLastError
#define hipStreamSynchronize cudaStreamSynchronize
#define hipGetErrorString cudaGetErrorString
#define hipGetErrorName cudaGetErrorName
/* HIP's unsynchronised wave shuffles, on a 32-wide wave */
#ifdef __CUDA_ARCH__
#define __shfl_xor(v, m) __shfl_xor_sync(0xffffffffu, (v), (m))
#define __shfl_down(v, d) __shfl_down_sync(0xffffffffu, (v), (d))
#endif


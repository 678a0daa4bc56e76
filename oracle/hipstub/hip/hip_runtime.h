/* hip/hip_runtime.h -- a stand-in that lets nvcc compile libr3d's HIP sources where they lie,
 * for the reference pin only (oracle/ref_band.cu). It maps the handful of HIP runtime names those
 * files use onto CUDA's.
 * TEST INFRASTRUCTURE ONLY. */
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>   /* before the shuffle macros below: NVIDIA's headers use the four-argument forms */
#include <mma.h>
#include <cstdint>
#include <cstring>

typedef cudaStream_t hipStream_t;
typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
#define hipGetLastError cudaGetLastError
#define hipStreamSynchronize cudaStreamSynchronize
#define hipGetErrorString cudaGetErrorString
#define hipGetErrorName cudaGetErrorName
#define hipGetDevice cudaGetDevice
#define hipStreamNonBlocking cudaStreamNonBlocking
#define hipStreamCreateWithFlags cudaStreamCreateWithFlags
#define hipStreamDestroy cudaStreamDestroy
#define hipDeviceSynchronize cudaDeviceSynchronize
#define hipMalloc cudaMalloc
#define hipFree cudaFree
#define hipMemGetInfo cudaMemGetInfo
#define hipMemcpyAsync cudaMemcpyAsync
#define hipMemsetAsync cudaMemsetAsync
#define hipFuncSetAttribute cudaFuncSetAttribute
#define hipFuncAttributeMaxDynamicSharedMemorySize cudaFuncAttributeMaxDynamicSharedMemorySize
/* hipLaunchKernelGGL((kernel<...>), grid, block, smem, stream, args...): the reference passes the
 * kernel in parentheses, which the <<< >>> syntax does not take, so the launch goes through a
 * function pointer */
template <typename... KArgs, typename... Args>
static inline void ref_launch_ggl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    kern<<<grid, block, smem, st>>>(args...);
}
#define hipLaunchKernelGGL(kern, grid, block, smem, stream, ...) \
    ref_launch_ggl(kern, dim3(grid), dim3(block), (size_t)(smem), (stream), __VA_ARGS__)
/* the reference gates its kernels on the chip's architecture name: the pin answers with the one
 * it expects, so that its own code paths run */
struct hipDeviceProp_t { char gcnArchName[256]; int multiProcessorCount; size_t totalGlobalMem; };
static inline cudaError_t hipGetDeviceProperties(hipDeviceProp_t* p, int dev) {
    cudaDeviceProp q;
    const cudaError_t e = cudaGetDeviceProperties(&q, dev);
    strcpy(p->gcnArchName, "gfx1100");
    p->multiProcessorCount = q.multiProcessorCount; p->totalGlobalMem = q.totalGlobalMem;
    return e;
}
/* Wave shuffles. HIP does not hold a *_sync shuffle to its mask argument the way CUDA does: the
 * reference's vectorised gated quantiser (src/r3d_band.hip:313 of libr3d) builds its mask from
 * threadIdx.x, which names the executing lane only in the first warp of a block; under CUDA's rule
 * ("every executing lane must be in the mask") that raised "illegal instruction" on B200. Every
 * shuffle of the pin builds therefore runs over the lanes that are active at the call, which is
 * what the HIP code relies on. */
#ifdef __CUDA_ARCH__
template <typename T> __device__ __forceinline__ T ref_shfl_xor_active(T v, int m) { return __shfl_xor_sync(__activemask(), v, m); }
template <typename T> __device__ __forceinline__ T ref_shfl_down_active(T v, unsigned d) { return __shfl_down_sync(__activemask(), v, d); }
#define __shfl_xor_sync(mask, v, m) ref_shfl_xor_active((v), (int)(m))
#define __shfl_down_sync(mask, v, d) ref_shfl_down_active((v), (unsigned)(d))
#define __shfl_xor(v, m) ref_shfl_xor_active((v), (int)(m))
#define __shfl_down(v, d) ref_shfl_down_active((v), (unsigned)(d))
#endif


/* AMD cross-lane and dot builtins the reference's mxfp4 file uses, with the same meaning on a
 * 32-wide warp: DPP row_xmask:k (control 0x160 | k) is "lane ^ k", permlanex16 with identity
 * selectors is "lane ^ 16", sudot4 with both operands signed is the signed byte dot. */
__device__ __forceinline__ int __builtin_amdgcn_update_dpp(int old, int src, int ctrl, int, int, bool) {
    (void)old;
    return __shfl_xor_sync(0xffffffffu, src, ctrl & 0xf);   /* -> active lanes, see above */
}
__device__ __forceinline__ unsigned __builtin_amdgcn_permlanex16(unsigned old, unsigned src, unsigned, unsigned, bool, bool) {
    (void)old;
    return __shfl_xor_sync(0xffffffffu, src, 16);
}
__device__ __forceinline__ int __builtin_amdgcn_sudot4(bool, int a, bool, int b, int c, bool) { return __dp4a(a, b, c); }
/* clang's streaming-load hint: a plain load has the same value. */
template <typename T> __host__ __device__ __forceinline__ T __builtin_nontemporal_load(const T* p) { return *p; }

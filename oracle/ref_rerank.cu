/* ref_rerank.cu -- libr3d's joined-e4m3 rerank file compiled from where it lies in the mounted
 * reference tree (never copied): src/r3d_logit_rerank_e4m3.hip, through nvcc for sm_100a with
 * oracle/hipstub standing in for the HIP headers and this repository's rad_*.h stand-ins for
 * radiance's. Its kernel is one thread per candidate with no warp-level builtins, so it runs on a
 * 32-wide NVIDIA warp as written. The reference reads the head's rad.planes header through the operand
 * pointer on the host, so the test keeps the head in managed memory. TEST INFRASTRUCTURE ONLY. */
#include <cuda_runtime.h>
#include <cstdint>
#include "r3d_logit_rerank_e4m3.hip"

void r3d_dump_begin(R3dDumpSlot* slot, const char*, const void*, const RadArgs*, RadStream) { if (slot) slot->priv = nullptr; }
void r3d_dump_end(R3dDumpSlot*, int) {}

#define REF_API extern "C" __attribute__((visibility("default")))
REF_API int ref_logit_rerank_e4m3(const RadArgs* a, void* stream) { return r3d_rad_logit_rerank_e4m3(a, (RadStream)stream); }
REF_API void* ref_rerank_alloc(long long bytes) {
    void* p = nullptr;
    return cudaMallocManaged(&p, (size_t)bytes) == cudaSuccess ? p : nullptr;
}
REF_API void ref_rerank_free(void* p) { (void)cudaFree(p); }

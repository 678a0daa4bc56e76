/* q8x_static.cu -- the int8-per-32 mxfp4a8 decode arm for callers that must not allocate.
 *
 * Who that is: a row's `launch` may be issued while the engine is recording a pass for later
 * replay, or after the engine has handed every byte of device memory to weights and KV cache.
 * In the first case a cudaMalloc would synchronise the device and break the recording; in
 * the second it simply fails. The ordinary arm (r3d_b200_gemm_mxfp4a8_q8x) leaves the
 * problem to its caller, who must bring the requantised-activation scratch. This entry point
 * brings its own: a fixed array that is part of the library image, so it exists on every
 * GPU from the moment the library is loaded there until the process ends, and no call ever
 * asks the allocator for anything.
 *
 * Limits and sharing rules (all follow from the array being one fixed, shared object):
 *   - M <= 8 tokens and K <= 32768 (K a multiple of 256, as the arm requires); larger
 *     calls are refused with RAD_E_SHAPE and a message, never truncated.
 *   - 288 KiB of device memory per GPU that loads the library, held until exit.
 *   - Every call on a device uses the same bytes. The requantise step overwrites the whole
 *     region the dot step then reads (M*K codes, M*K/32 scales), so nothing has to start at
 *     zero and nothing of an earlier call leaks into a later one -- but two calls that
 *     overlap in time on one device (different streams, or two host threads) race on it.
 *     Issue them on one stream, or order them with events.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, no allocation). Make that first call before any stream capture
 *     begins on that device.
 */
#include <cstdio>
#include "r3d_kernels.h"

constexpr int kMaxTokens = 8;
constexpr int kMaxK = 32768;
constexpr size_t kCodeBytes = (size_t)kMaxTokens * kMaxK;                    /* int8 x8[M][K] */
constexpr size_t kScaleBytes = (size_t)kMaxTokens * (kMaxK / 32) * sizeof(float);
constexpr int kMaxDevices = 64;

/* In host code this name is only a handle for the runtime; the usable device pointer is
 * whatever cudaGetSymbolAddress returns for the current device. */
static __device__ __align__(256) unsigned char g_q8x_scratch[kCodeBytes + kScaleBytes];

namespace {

unsigned char* scratch_on_current_device() {
    static unsigned char* known[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!known[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_q8x_scratch);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "libr3d_b200: no device address for the built-in q8x scratch on "
                            "device %d (%s)\n", dev, cudaGetErrorString(e));
            return nullptr;
        }
        known[dev] = (unsigned char*)p;
    }
    return known[dev];
}

} /* namespace */

extern "C" int r3d_b200_gemm_mxfp4a8_q8x_static(const R3dGemmQ* q, int walk, void* stream) {
    if (!q) return RAD_E_INVAL;
    if (!r3d::device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (q->m < 1 || q->k < 256 || (q->k & 255)) return RAD_E_UNSUPPORTED;
    if (q->m > kMaxTokens || q->k > kMaxK) {
        fprintf(stderr, "libr3d_b200: q8x_static serves at most M=%d, K=%d (got M=%d, K=%d); "
                        "use r3d_b200_gemm_mxfp4a8_q8x with caller scratch\n",
                kMaxTokens, kMaxK, q->m, q->k);
        return RAD_E_SHAPE;
    }
    unsigned char* base = scratch_on_current_device();
    if (!base) return RAD_E_DEVICE;
    int8_t* x8 = (int8_t*)base;
    float* sg = (float*)(base + kCodeBytes);
    cudaStream_t st = (cudaStream_t)stream;
    return r3d::q8x_run(*q, x8, sg, walk ? 1 : 0, st);
}

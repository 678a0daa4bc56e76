/* planes_cache.cpp -- host-readable copies of rad.planes headers that live in device memory.
 *
 * The reference reads a joined-weight blob's header through the operand pointer on the host at every
 * call (src/r3d_gemm_logits.hip:176-194, src/r3d_gemm_w2a8.hip:1010-1028 of libr3d), which works where
 * device memory is host-visible. A CUDA device allocation is not, so the header and entry table of a
 * device-resident blob are copied to the host once, on first sight of that pointer, and remembered
 * (weights are immortal for the life of the engine). That first call synchronises; later calls do
 * not. The engine may still put another blob at the same address (a reload, a caching allocator):
 * callers re-read once before they refuse on a remembered header, and r3d_b200_forget_head drops one. */
#include <vector>
#include <cuda_runtime.h>
#include "entry_util.h"
#include "rad_planes.h"
#include "r3d_b200.h"

namespace r3d {

namespace {
struct HeadView {
    const void* blob;               /* key: the operand's data pointer */
    alignas(16) unsigned char head[sizeof(RadPlanesHeader) +
                                   RAD_ENC_MAX_PLANES * sizeof(RadPlanesEntry)];
};
std::vector<HeadView*>& seen_heads() { static std::vector<HeadView*> v; return v; }

bool read_head(HeadView* v) {
    cudaPointerAttributes at{};
    const bool have = cudaPointerGetAttributes(&at, v->blob) == cudaSuccess;
    if (!have) (void)cudaGetLastError();
    if (have && at.type == cudaMemoryTypeDevice) {
        if (cudaMemcpy(v->head, v->blob, sizeof v->head, cudaMemcpyDeviceToHost) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    } else {
        memcpy(v->head, v->blob, sizeof v->head);   /* host, pinned or managed memory */
    }
    return true;
}
} /* namespace */

const unsigned char* planes_head_of(const void* blob, bool* cached) {
    for (const HeadView* v : seen_heads()) if (v->blob == blob) { *cached = true; return v->head; }
    *cached = false;
    HeadView* v = new HeadView;
    v->blob = blob;
    if (!read_head(v)) { delete v; return nullptr; }
    seen_heads().push_back(v);
    return v->head;
}

const unsigned char* planes_head_refresh(const void* blob) {
    for (HeadView* v : seen_heads()) if (v->blob == blob) return read_head(v) ? v->head : nullptr;
    return nullptr;
}

} /* namespace r3d */

extern "C" void r3d_b200_forget_head(const void* blob) {
    std::vector<r3d::HeadView*>& v = r3d::seen_heads();
    for (size_t i = 0; i < v.size(); ++i)
        if (v[i]->blob == blob) { delete v[i]; v.erase(v.begin() + (long)i); return; }
}

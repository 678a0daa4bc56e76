/* push.cuh -- the all-gather of a column-sharded GEMV fused into its epilogue.
 *
 * Every rank owns a slab of weight rows (= output columns). Instead of writing its slab to a
 * local y and calling a collective, the kernel's epilogue stores each output element straight
 * into the gathered [M, world * n_pad] buffer of every rank (its own included) through peer
 * mappings of those buffers (plain st.global over NVLink; no remote loads). The kernel does not
 * signal: the kernel that follows it in the stream (k_gather_wait) starts when the GEMV grid has
 * completed, publishes this rank's call count to every rank's flag array by release stores at
 * system scope, and then waits (bounded, acquire loads) until every rank's count has reached
 * its own. Ranks issue the same sequence of calls, so the counts agree without host traffic and
 * survive graph replay.
 * (Signalling from the GEMV itself needs a fence per CTA, which queues behind the weight
 * stream: measured +4.5 to +17 us per call depending on where the fences sit.) */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace r3d {

constexpr int kMaxRanks = 8;

struct PushCfg {
    void* dst[kMaxRanks];          /* the gathered buffer (this call's slot) on every rank */
    int64_t pitch;                 /* elements per gathered row: world * n_pad */
    int64_t col0;                  /* rank * n_pad */
    int world;                     /* 0: no push, the kernel stores to its own y */
};

template <typename T>
__device__ __forceinline__ void push_store(const PushCfg& g, int t, int col, T v) {
    const int64_t at = (int64_t)t * g.pitch + g.col0 + col;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
        if (p < g.world) ((T*)g.dst[p])[at] = v;
}

} /* namespace r3d */

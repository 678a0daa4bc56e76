/* push.cuh -- the all-gather of a column-sharded GEMV fused into its epilogue.
 *
 * Every rank owns a slab of weight rows (= output columns). Instead of writing its slab to a
 * local y and calling a collective, the kernel's epilogue stores each output element straight
 * into the gathered [M, world * n_pad] buffer of every rank (its own included) through peer
 * mappings of those buffers (plain st.global over NVLink; no remote loads). When the last CTA of
 * the grid has stored, it raises this rank's flag word in every rank's flag array to the number
 * of pushes this rank has completed. A consumer waits (k_gather_wait, bounded) until all flags
 * have reached its own count of calls: ranks issue the same sequence of calls, so the counts
 * agree without any host traffic and survive CUDA-graph replay. */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace r3d {

constexpr int kMaxRanks = 8;

struct PushCfg {
    void* dst[kMaxRanks];          /* the gathered buffer (this call's slot) on every rank */
    uint32_t* flag[kMaxRanks];     /* this rank's flag word on every rank */
    uint32_t* counter;             /* local: CTAs of the running grid that have stored (resets itself) */
    uint32_t* epoch;               /* local: pushes this rank has completed */
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

/* One thread per CTA, after every storing thread of the CTA has executed __threadfence_system()
 * and the CTA has synchronised. */
__device__ __forceinline__ void push_signal(const PushCfg& g) {
    __threadfence_system();
    const uint32_t done = atomicAdd(g.counter, 1u);
    if (done == gridDim.x * gridDim.y * gridDim.z - 1u) {
        *g.counter = 0u;
        __threadfence_system();
        const uint32_t e = atomicAdd(g.epoch, 1u) + 1u;
        for (int p = 0; p < g.world; ++p) *(volatile uint32_t*)g.flag[p] = e;
        __threadfence_system();
    }
}

} /* namespace r3d */

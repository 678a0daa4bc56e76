/* gather.cu -- host side of the fused GEMV + all-gather: the exchange buffers, their CUDA IPC
 * handles, the peer mappings and the bounded wait kernel. One process per GPU; the handles travel
 * between processes by whatever the host program uses (the Python package sends them through
 * torch.distributed). No reference counterpart: the reference is single-rank
 * (src/r3d_rows.cpp:281-284 of libr3d). */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include "r3d_kernels.h"
#include "push.cuh"

namespace r3d {

struct Gather {
    int world, rank, slots;
    int64_t slot_bytes;
    uint8_t* local;                    /* [flag word per rank: 256 B][epoch, status: 256 B][slots x slot_bytes] */
    uint8_t* peer[kMaxRanks];          /* peer[rank] == local */
    bool opened[kMaxRanks];
};

namespace {
constexpr int64_t kHdr = 512;      /* [0,256): flag word per rank; [256,512): epoch, status */

struct FlagPtrs { uint32_t* p[kMaxRanks]; };

/* Runs after the pushing kernel of the same call. It may be made resident early (programmatic
 * stream serialisation) and lets its own successor be scheduled at once, but does nothing before
 * the pushing grid has completed and flushed. Then thread p stores this rank's call count into
 * its flag word on rank p with release semantics at system scope and polls rank p's word here
 * with acquire loads, bounded. (A system fence, a plain store, a volatile poll and a second fence
 * do the same and measured 2 us more per call on two GPUs: the second fence waits for the flag
 * store's own round trip over NVLink.) */
__global__ void k_gather_wait(const uint32_t* flags, FlagPtrs mine, uint32_t* epoch, int* status, int world) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    /* every thread reads the count itself: the grid is one warp, and the word is rewritten only
     * after all of them have read it */
    const uint32_t want = *(volatile uint32_t*)epoch + 1u;
    __syncwarp();
    if (threadIdx.x == 0) *epoch = want;
    if ((int)threadIdx.x < world) {
        /* release: the pushing grid's stores, visible to this thread since the dependency wait,
         * are performed at the peer before the count is */
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(mine.p[threadIdx.x]), "r"(want) : "memory");
        const long long t0 = clock64();
        for (;;) {
            /* acquire: what follows (this kernel's end, then the readers of the gathered buffer)
             * is ordered after the observation, as the peer's stores were ordered before its count */
            uint32_t got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(flags + threadIdx.x) : "memory");
            if ((int)(got - want) >= 0) break;
            if (clock64() - t0 > 2000000000LL) { atomicExch(status, 1 + (int)threadIdx.x); break; }
        }
    }
    /* kernels that follow in the stream read the gathered buffer from this GPU's own memory,
     * where the peers' stores have landed before their flag did */
}
} /* namespace */

bool gather_push_cfg(const Gather* g, int slot, int64_t n_pad, int m, int elem_bytes, PushCfg* out) {
    if (!g || slot < 0 || slot >= g->slots || n_pad <= 0 || m <= 0) return false;
    if ((int64_t)m * g->world * n_pad * elem_bytes > g->slot_bytes) return false;
    PushCfg c{};
    for (int p = 0; p < g->world; ++p) {
        if (!g->peer[p]) return false;
        c.dst[p] = g->peer[p] + kHdr + (int64_t)slot * g->slot_bytes;
    }
    c.pitch = n_pad * g->world;
    c.col0 = n_pad * g->rank;
    c.world = g->world;
    *out = c;
    return true;
}

namespace {
/* the unfused form: copy a finished [m, n] slab into every rank's gathered buffer, then signal */
template <typename T>
__global__ void k_push_copy(const T* __restrict__ y, int64_t y_pitch, int m, int n, const PushCfg g) {
    const int64_t total = (int64_t)m * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), c = (int)(i - (int64_t)t * n);
        push_store<T>(g, t, c, y[(int64_t)t * y_pitch + c]);
    }
    __syncthreads();
}
} /* namespace */

int push_copy(const void* y, int64_t y_pitch, int m, int n, int elem_bytes, const PushCfg& g, cudaStream_t st) {
    const int64_t total = (int64_t)m * n;
    const int blocks = (int)((total + 255) / 256 < 592 ? (total + 255) / 256 : 592);
    count_launch();
    if (elem_bytes == 4) k_push_copy<float><<<blocks, 256, 0, st>>>((const float*)y, y_pitch, m, n, g);
    else k_push_copy<uint16_t><<<blocks, 256, 0, st>>>((const uint16_t*)y, y_pitch, m, n, g);
    return cudaGetLastError() == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

} /* namespace r3d */

using namespace r3d;

extern "C" {

int r3d_b200_gather_create(int world, int rank, int64_t slot_bytes, int slots, void** out,
                           unsigned char handle[64]) {
    if (!out || !handle || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slots < 1 ||
        slot_bytes <= 0) return RAD_E_INVAL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    Gather* g = new (std::nothrow) Gather();
    if (!g) return RAD_E_DEVICE;
    g->world = world; g->rank = rank; g->slots = slots;
    g->slot_bytes = (slot_bytes + 255) / 256 * 256;
    const size_t bytes = (size_t)(kHdr + g->slot_bytes * slots);
    if (cudaMalloc((void**)&g->local, bytes) != cudaSuccess || cudaMemset(g->local, 0, bytes) != cudaSuccess) {
        (void)cudaGetLastError(); delete g; return RAD_E_DEVICE;
    }
    for (int p = 0; p < kMaxRanks; ++p) { g->peer[p] = nullptr; g->opened[p] = false; }
    g->peer[rank] = g->local;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, g->local) != cudaSuccess) { (void)cudaGetLastError(); cudaFree(g->local); delete g; return RAD_E_DEVICE; }
    memcpy(handle, &h, 64);
    if (cudaDeviceSynchronize() != cudaSuccess) { (void)cudaGetLastError(); }
    *out = g;
    return RAD_OK;
}

/* handles: world x 64 bytes, rank-major (this rank's own entry is ignored) */
int r3d_b200_gather_connect(void* gp, const unsigned char* handles) {
    Gather* g = (Gather*)gp;
    if (!g || !handles) return RAD_E_INVAL;
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank || g->peer[p]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * p, 64);
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            return RAD_E_DEVICE;
        }
        g->peer[p] = (uint8_t*)ptr; g->opened[p] = true;
    }
    return RAD_OK;
}

/* A peer that lives in the same process (one process driving several GPUs with peer access
 * enabled, or a test): hand over the base pointer of its exchange buffer instead of a handle. */
int r3d_b200_gather_connect_ptr(void* gp, int peer, void* base) {
    Gather* g = (Gather*)gp;
    if (!g || !base || peer < 0 || peer >= g->world || peer == g->rank) return RAD_E_INVAL;
    g->peer[peer] = (uint8_t*)base; g->opened[peer] = false;
    return RAD_OK;
}

void* r3d_b200_gather_base(void* gp) { return gp ? ((Gather*)gp)->local : nullptr; }

/* this rank's gathered buffer of a slot: [M, world * n_pad] elements once all ranks have pushed */
void* r3d_b200_gather_buffer(void* gp, int slot) {
    Gather* g = (Gather*)gp;
    if (!g || slot < 0 || slot >= g->slots) return nullptr;
    return g->local + kHdr + (int64_t)slot * g->slot_bytes;
}

/* enqueue the wait for every rank's next push; at most ~1 s on the device, then status != 0 */
int r3d_b200_gather_wait(void* gp, void* stream) {
    Gather* g = (Gather*)gp;
    if (!g) return RAD_E_INVAL;
    count_launch();
    FlagPtrs mine{};
    for (int p = 0; p < g->world; ++p) {
        if (!g->peer[p]) return RAD_E_INVAL;
        mine.p[p] = (uint32_t*)g->peer[p] + g->rank;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool off = [] { const char* e = getenv("R3D_NO_PDL"); return e && *e && *e != '0'; }();
    cfg.attrs = at; cfg.numAttrs = off ? 0 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, k_gather_wait, (const uint32_t*)g->local, mine,
                                             (uint32_t*)(g->local + 256), (int*)(g->local + 256) + 1, g->world);
    return e == cudaSuccess ? RAD_OK : RAD_E_DEVICE;
}

/* 0, or 1 + the rank whose push did not arrive within the wait's limit (synchronises the device) */
int r3d_b200_gather_status(void* gp) {
    Gather* g = (Gather*)gp;
    if (!g) return -1;
    int v = 0;
    if (cudaMemcpy(&v, (int*)(g->local + 256) + 1, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return v;
}

void r3d_b200_gather_destroy(void* gp) {
    Gather* g = (Gather*)gp;
    if (!g) return;
    for (int p = 0; p < g->world; ++p)
        if (g->opened[p]) (void)cudaIpcCloseMemHandle(g->peer[p]);
    (void)cudaFree(g->local);
    delete g;
}

} /* extern "C" */

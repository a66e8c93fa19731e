// Shared helpers for the sm_100a kernels behind include/ogle_cuda.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include "ogle_cuda.h"

namespace ogle {

extern std::atomic<uint64_t> g_launch_count;
void set_last_error(cudaError_t e);
void set_last_error(const char* message);

// B200: 148 SMs. Grid-stride kernels launch a multiple of this.
constexpr int kNumSMs = 148;

inline int up4(int v) { return (v + 3) / 4 * 4; }
inline int div_up(long a, long b) { return int((a + b - 1) / b); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks the launch just made; counts it.
inline int finish_launch() {
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        set_last_error(e);
        (void)cudaGetLastError();
        return OGLE_ERR_CUDA;
    }
    return OGLE_OK;
}

// Grid size for a grid-stride loop over `items` work items with `threads` per
// block: enough blocks to cover the work, capped at 8 resident blocks per SM.
inline int grid_for(long items, int threads, int max_per_sm = 8) {
    long blocks = (items + threads - 1) / threads;
    long cap = long(kNumSMs) * max_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return int(blocks);
}

// Programmatic dependent launch. A kernel launched through launch_overlapped() may be scheduled while
// the kernel before it on the stream is still running: its blocks start as that kernel's blocks retire,
// do their set-up (shared-memory barriers, tensor-memory allocation, index tables) and only then wait
// for the predecessor's results. Every kernel launched that way calls grid_dependency_wait() before its
// first access to global memory that another kernel may write or read, and
// grid_dependency_trigger() at its top, which lets ITS successor be scheduled early in turn. Both are
// no-ops in a kernel launched the ordinary way. In a captured graph the dependency becomes a programmatic
// edge; a predecessor that is not a kernel (memset, copy, event wait) keeps an ordinary, full dependency.
// Off by default (every launch is then an ordinary one); OGLE_PDL=1 turns it on.
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool overlapped_launches_enabled();
void set_overlapped_launches(int on);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlapped_launches_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float apply_act(float v, int act, float lo, float hi) {
    // conv2d.glsl:82-90: clip is min(max(v,lo),hi), relu is max(0,v)
    if (act == OGLE_ACT_CLIP) return fminf(fmaxf(v, lo), hi);
    if (act == OGLE_ACT_RELU) return fmaxf(v, 0.f);
    return v;
}

__device__ __forceinline__ float4 apply_act4(float4 v, int act, float lo, float hi) {
    v.x = apply_act(v.x, act, lo, hi);
    v.y = apply_act(v.y, act, lo, hi);
    v.z = apply_act(v.z, act, lo, hi);
    v.w = apply_act(v.w, act, lo, hi);
    return v;
}

}  // namespace ogle

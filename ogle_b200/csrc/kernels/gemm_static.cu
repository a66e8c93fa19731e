// ogle_cuda_gemm_static: the run-time-B tensor-core GEMM with its packing scratch in a
// file-scope device array, for callers that may not allocate device memory and have no
// workspace of their own to lend. No counterpart in the reference.
//
// Set-up happens on the FIRST call per device, with that device current: the address of the
// array is resolved with cudaGetSymbolAddress and cached. Make that first call before any
// stream capture. Later calls only launch kernels.
//
// The array is shared by every call in the process on that device. The packing pass rewrites
// every byte the multiply later reads (padding included), so nothing has to start at zero;
// but two calls whose execution may overlap (different streams, or different host threads
// without ordering) race on the array. Order them on one stream or with events.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "common.cuh"
#include "ogle_cuda.h"

namespace {

constexpr size_t kScratchBytes = OGLE_GEMM_STATIC_MAX_BYTES;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_gemm_scratch[kScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Resolves (once per device) the device address of the scratch array for the current device.
int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        ogle::set_last_error("gemm_static: cannot identify the current device");
        return OGLE_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_gemm_scratch);
        if (e != cudaSuccess || !ptr) {
            ogle::set_last_error((std::string("gemm_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e)).c_str());
            return OGLE_ERR_CUDA;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return OGLE_OK;
}

}  // namespace

extern "C" size_t ogle_cuda_gemm_static_max_bytes(void) { return kScratchBytes; }

extern "C" int ogle_cuda_gemm_static(const OgleGemmParams* p, const float* A, const float* B, const float* C, float* Y,
                                     ogle_stream_t stream) {
    if (!p) return OGLE_ERR_INVALID;
    if (p->math_mode == OGLE_MATH_FP32) return ogle_cuda_gemm(p, A, B, C, Y, stream);   // needs no scratch
    const size_t need = ogle_cuda_gemm_packed_b_bytes(p);
    if (need == 0) return OGLE_ERR_INVALID;
    if (need > kScratchBytes) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "gemm_static: packed B needs %zu bytes, the static scratch holds %zu; use ogle_cuda_gemm_ws with a "
                 "caller-owned workspace", need, kScratchBytes);
        ogle::set_last_error(msg);
        return OGLE_ERR_UNSUPPORTED;
    }
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != OGLE_OK) return rc;
    return ogle_cuda_gemm_ws(p, A, B, C, Y, scratch, kScratchBytes, stream);
}

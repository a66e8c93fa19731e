// Max / average / global-average pooling over NHWC4 activations.
//
// HBM-bound: algorithmic traffic is the input read once plus the output written
// once. One thread owns 4 channels (a float4) of a TY x TX patch of output
// pixels and walks the input rows of that patch once, so that the overlap of
// neighbouring windows is reused from registers instead of re-read through L1/L2.
// Channels are the fastest-varying thread index, so a warp reads and writes
// 512-byte contiguous runs.
#include <cfloat>
#include "common.cuh"

namespace ogle {

struct PoolArgs {
    int N, H, W, C4, Ho, Wo;      // C4 = float4s per pixel that hold real channels
    int in_q, out_q;              // float4s per pixel (channel stride / 4)
    int kernel, stride, pad, type;
};

__device__ __forceinline__ float4 f4max(float4 a, float4 b) {
    return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
}
__device__ __forceinline__ float4 f4add(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// Index: the type the item index is split in (32-bit when the item count allows: the three
// divisions per item cost more in 64 bits than the patch's max/add work).
template <int K, int S, int TY, int TX, bool MAX, typename Index>
__global__ void pool_patch_kernel(const float4* __restrict__ x, float4* __restrict__ y, PoolArgs a) {
    constexpr int PH = (TY - 1) * S + K, PW = (TX - 1) * S + K;
    const int gy = (a.Ho + TY - 1) / TY, gx = (a.Wo + TX - 1) / TX;
    const Index total = (Index)a.N * gy * gx * a.C4;
    const float init = MAX ? -FLT_MAX : 0.f;
    const Index step = (Index)gridDim.x * blockDim.x;
    for (Index i = blockIdx.x * (Index)blockDim.x + threadIdx.x; i < total; i += step) {
        Index t = i;
        const int c4 = int(t % a.C4); t /= a.C4;
        const int px = int(t % gx); t /= gx;
        const int py = int(t % gy); t /= gy;
        const int n = int(t);
        const int oy0 = py * TY, ox0 = px * TX;
        const int iy0 = oy0 * S - a.pad, ix0 = ox0 * S - a.pad;
        float4 acc[TY][TX];
#pragma unroll
        for (int ty = 0; ty < TY; ++ty)
#pragma unroll
            for (int tx = 0; tx < TX; ++tx) acc[ty][tx] = make_float4(init, init, init, init);
#pragma unroll
        for (int r = 0; r < PH; ++r) {
            const int iy = iy0 + r;
            if (iy < 0 || iy >= a.H) continue;
            const float4* row = x + ((long)n * a.H + iy) * a.W * a.in_q + c4;
            float4 v[PW];
#pragma unroll
            for (int c = 0; c < PW; ++c) {
                const int ix = ix0 + c;
                v[c] = (ix >= 0 && ix < a.W) ? row[(long)ix * a.in_q] : make_float4(init, init, init, init);
            }
#pragma unroll
            for (int ty = 0; ty < TY; ++ty) {
                if (r < ty * S || r >= ty * S + K) continue;
#pragma unroll
                for (int tx = 0; tx < TX; ++tx)
#pragma unroll
                    for (int kx = 0; kx < K; ++kx)
                        acc[ty][tx] = MAX ? f4max(acc[ty][tx], v[tx * S + kx]) : f4add(acc[ty][tx], v[tx * S + kx]);
            }
        }
#pragma unroll
        for (int ty = 0; ty < TY; ++ty)
#pragma unroll
            for (int tx = 0; tx < TX; ++tx) {
                const int oy = oy0 + ty, ox = ox0 + tx;
                if (oy >= a.Ho || ox >= a.Wo) continue;
                float4 r = acc[ty][tx];
                if (MAX) {
                    // a window that holds only padding yields 0 (pool.glsl:28-29)
                    if (r.x == -FLT_MAX) r.x = 0.f;
                    if (r.y == -FLT_MAX) r.y = 0.f;
                    if (r.z == -FLT_MAX) r.z = 0.f;
                    if (r.w == -FLT_MAX) r.w = 0.f;
                } else {
                    const float d = float(K * K);  // padding counts (pool.glsl:62-65)
                    r = make_float4(r.x / d, r.y / d, r.z / d, r.w / d);
                }
                y[(((long)n * a.Ho + oy) * a.Wo + ox) * a.out_q + c4] = r;
            }
    }
}

// Any kernel/stride: one thread per output float4, loops over the window.
__global__ void pool_generic_kernel(const float4* __restrict__ x, float4* __restrict__ y, PoolArgs a) {
    const long total = (long)a.N * a.Ho * a.Wo * a.C4;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int c4 = int(t % a.C4); t /= a.C4;
        const int ox = int(t % a.Wo); t /= a.Wo;
        const int oy = int(t % a.Ho); t /= a.Ho;
        const int n = int(t);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        bool first = true;
        for (int kx = 0; kx < a.kernel; ++kx)
            for (int ky = 0; ky < a.kernel; ++ky) {  // pool.glsl:31-32: columns outer, rows inner
                const int ix = ox * a.stride + kx - a.pad, iy = oy * a.stride + ky - a.pad;
                if (ix < 0 || ix >= a.W || iy < 0 || iy >= a.H) continue;
                const float4 v = x[(((long)n * a.H + iy) * a.W + ix) * a.in_q + c4];
                if (a.type == 0) {
                    acc = first ? v : f4max(acc, v);
                    first = false;
                } else {
                    acc = f4add(acc, v);
                }
            }
        if (a.type != 0) {
            const float d = float(a.kernel * a.kernel);
            acc = make_float4(acc.x / d, acc.y / d, acc.z / d, acc.w / d);
        }
        y[(((long)n * a.Ho + oy) * a.Wo + ox) * a.out_q + c4] = acc;
    }
}

// Global average: one warp per (image, float4 of channels); lanes stride over the
// pixels and combine with shuffles. The sum order differs from the reference's
// serial loop; results agree to fp32 rounding of a k*k-term sum.
__global__ void pool_global_kernel(const float4* __restrict__ x, float4* __restrict__ y, PoolArgs a) {
    const int lane = threadIdx.x & 31;
    const long warp = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
    const long total = (long)a.N * a.C4;
    const int hw = a.H * a.W;
    for (long w = warp; w < total; w += nwarps) {
        const int c4 = int(w % a.C4);
        const int n = int(w / a.C4);
        const float4* base = x + (long)n * hw * a.in_q + c4;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = lane; p < hw; p += 32) s = f4add(s, base[(long)p * a.in_q]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s.x += __shfl_xor_sync(0xffffffffu, s.x, o);
            s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
            s.z += __shfl_xor_sync(0xffffffffu, s.z, o);
            s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
        }
        if (lane == 0) {
            const float d = float(a.kernel * a.kernel);
            y[(long)n * a.out_q + c4] = make_float4(s.x / d, s.y / d, s.z / d, s.w / d);
        }
    }
}

}  // namespace ogle

using namespace ogle;

extern "C" {

int ogle_cuda_pool_infer(OglePoolParams* p) {
    if (!p) return OGLE_ERR_INVALID;
    const int H = p->in_hwc[0], W = p->in_hwc[1], C = p->in_hwc[2];
    if (p->N <= 0 || H <= 0 || W <= 0 || C <= 0) return OGLE_ERR_INVALID;
    if (p->type == 2) {
        // pool.cc:84-91: kernel := H, stride 1, pad 0, requires a square map
        if (H != W) return OGLE_ERR_UNSUPPORTED;
        p->kernel = H; p->stride = 1; p->pad = 0;
        p->out_hwc[0] = 1; p->out_hwc[1] = 1; p->out_hwc[2] = C;
        return OGLE_OK;
    }
    if (p->kernel <= 0 || p->stride <= 0 || p->pad < 0) return OGLE_ERR_INVALID;
    p->out_hwc[0] = (H - p->kernel + 2 * p->pad) / p->stride + 1;  // pool.cc:93-96
    p->out_hwc[1] = (W - p->kernel + 2 * p->pad) / p->stride + 1;
    p->out_hwc[2] = C;
    if (p->out_hwc[0] <= 0 || p->out_hwc[1] <= 0) return OGLE_ERR_INVALID;
    return OGLE_OK;
}

int ogle_cuda_pool(const OglePoolParams* p, const float* x, float* y, ogle_stream_t stream) {
    if (!p || !x || !y) return OGLE_ERR_INVALID;
    OglePoolParams q = *p;
    int rc = ogle_cuda_pool_infer(&q);
    if (rc != OGLE_OK) return rc;
    if (q.out_hwc[0] != p->out_hwc[0] || q.out_hwc[1] != p->out_hwc[1] || q.out_hwc[2] != p->out_hwc[2])
        return OGLE_ERR_INVALID;
    if (q.type < 0 || q.type > 2) return OGLE_ERR_INVALID;
    const int C = q.in_hwc[2];
    const int ics = q.in_channel_stride ? q.in_channel_stride : up4(C);
    const int ocs = q.out_channel_stride ? q.out_channel_stride : up4(C);
    if (ics < up4(C) || ocs < up4(C) || (ics & 3) || (ocs & 3)) return OGLE_ERR_INVALID;
    if (!aligned16(x) || !aligned16(y)) return OGLE_ERR_ALIGNMENT;
    PoolArgs a;
    a.N = q.N; a.H = q.in_hwc[0]; a.W = q.in_hwc[1]; a.C4 = up4(C) / 4;
    a.Ho = q.out_hwc[0]; a.Wo = q.out_hwc[1];
    a.in_q = ics / 4; a.out_q = ocs / 4;
    a.kernel = q.kernel; a.stride = q.stride; a.pad = q.pad; a.type = q.type;
    const float4* xi = reinterpret_cast<const float4*>(x);
    float4* yo = reinterpret_cast<float4*>(y);
    cudaStream_t s = (cudaStream_t)stream;
    if (q.type == 2 || (q.type == 1 && a.Ho == 1 && a.Wo == 1 && q.pad == 0 && q.kernel == a.H && q.kernel == a.W)) {
        const long warps = (long)a.N * a.C4;
        pool_global_kernel<<<grid_for(warps * 32, 256), 256, 0, s>>>(xi, yo, a);
    } else if (q.kernel == 3 && q.stride == 2) {
        const long items = (long)a.N * ((a.Ho + 1) / 2) * ((a.Wo + 1) / 2) * a.C4;
        const bool small = items < (1L << 30);
        const int grid = grid_for(items, 128, 16);
        if (q.type == 0 && small) pool_patch_kernel<3, 2, 2, 2, true, unsigned><<<grid, 128, 0, s>>>(xi, yo, a);
        else if (q.type == 0) pool_patch_kernel<3, 2, 2, 2, true, long><<<grid, 128, 0, s>>>(xi, yo, a);
        else if (small) pool_patch_kernel<3, 2, 2, 2, false, unsigned><<<grid, 128, 0, s>>>(xi, yo, a);
        else pool_patch_kernel<3, 2, 2, 2, false, long><<<grid, 128, 0, s>>>(xi, yo, a);
    } else if (q.kernel == 2 && q.stride == 2) {
        const long items = (long)a.N * a.Ho * ((a.Wo + 1) / 2) * a.C4;
        const bool small = items < (1L << 30);
        const int grid = grid_for(items, 128, 16);
        if (q.type == 0 && small) pool_patch_kernel<2, 2, 1, 2, true, unsigned><<<grid, 128, 0, s>>>(xi, yo, a);
        else if (q.type == 0) pool_patch_kernel<2, 2, 1, 2, true, long><<<grid, 128, 0, s>>>(xi, yo, a);
        else if (small) pool_patch_kernel<2, 2, 1, 2, false, unsigned><<<grid, 128, 0, s>>>(xi, yo, a);
        else pool_patch_kernel<2, 2, 1, 2, false, long><<<grid, 128, 0, s>>>(xi, yo, a);
    } else {
        const long items = (long)a.N * a.Ho * a.Wo * a.C4;
        pool_generic_kernel<<<grid_for(items, 256), 256, 0, s>>>(xi, yo, a);
    }
    return finish_launch();
}

}  // extern "C"

// Elementwise kernels (relu, clip, add, batchnorm): HBM-bound, 128-bit accesses,
// grid-stride over a grid that is a multiple of the SM count.
#include "common.cuh"

namespace ogle {

enum { EW_RELU = 0, EW_CLIP = 1, EW_ADD = 2, EW_ADD_RELU = 3, EW_ADD_CLIP = 4 };

template <int OP>
__global__ void elementwise_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                   float4* __restrict__ y, long n4, float lo, float hi) {
    grid_dependency_trigger();
    grid_dependency_wait();
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4;
         i += (long)gridDim.x * blockDim.x) {
        float4 v = a[i];
        if (OP == EW_ADD_RELU || OP == EW_ADD_CLIP) {
            // binary.glsl then relu.glsl / clip.glsl in one pass: the sum is rounded to fp32 before the
            // activation exactly as when it goes through memory, so the result is bit-identical
            const float4 w = b[i];
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        if (OP == EW_RELU || OP == EW_ADD_RELU) {
            v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
        } else if (OP == EW_CLIP || OP == EW_ADD_CLIP) {
            // clip.glsl:8-9: min(hi, max(lo, v))
            v.x = fminf(hi, fmaxf(lo, v.x)); v.y = fminf(hi, fmaxf(lo, v.y));
            v.z = fminf(hi, fmaxf(lo, v.z)); v.w = fminf(hi, fmaxf(lo, v.w));
        } else if (OP == EW_ADD) {
            const float4 w = b[i];
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        y[i] = v;
    }
}

// (x-mean)/sqrt(var+eps)*gamma+beta, evaluated in that order with IEEE divide and
// sqrt as batchnorm.glsl:31 writes it (not folded into scale/shift), so results
// match the reference's to the last bit per operation.
__global__ void batchnorm_kernel(const float4* __restrict__ x, const float* __restrict__ gamma,
                                 const float* __restrict__ beta, const float* __restrict__ mean,
                                 const float* __restrict__ var, float4* __restrict__ y,
                                 long pixels, int C, int q, float eps) {
    const long total = pixels * q;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int c = int(i % q) * 4;
        const float4 v = x[i];
        float in[4] = {v.x, v.y, v.z, v.w};
        float out[4];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            if (c + l < C) {
                const float d = __fsqrt_rn(__fadd_rn(var[c + l], eps));
                const float t = __fdiv_rn(__fsub_rn(in[l], mean[c + l]), d);
                out[l] = __fadd_rn(__fmul_rn(t, gamma[c + l]), beta[c + l]);
            } else {
                out[l] = 0.f;
            }
        }
        y[i] = make_float4(out[0], out[1], out[2], out[3]);
    }
}

}  // namespace ogle

using namespace ogle;

template <int OP>
static int launch_elementwise(const float* a, const float* b, float* y, long n, float lo, float hi,
                              ogle_stream_t stream) {
    if (n < 0 || (n & 3)) return OGLE_ERR_INVALID;
    if (n == 0) return OGLE_OK;
    if (!a || !y || (OP >= EW_ADD && !b)) return OGLE_ERR_INVALID;
    if (!aligned16(a) || !aligned16(y) || (b && !aligned16(b))) return OGLE_ERR_ALIGNMENT;
    launch_overlapped(elementwise_kernel<OP>, dim3(grid_for(n / 4, 256)), dim3(256), 0, (cudaStream_t)stream,
                      reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b), reinterpret_cast<float4*>(y), n / 4,
                      lo, hi);
    return finish_launch();
}

extern "C" {

int ogle_cuda_relu(const float* x, float* y, long n, ogle_stream_t stream) {
    return launch_elementwise<EW_RELU>(x, nullptr, y, n, 0.f, 0.f, stream);
}
int ogle_cuda_clip(const float* x, float* y, long n, float lo, float hi, ogle_stream_t stream) {
    return launch_elementwise<EW_CLIP>(x, nullptr, y, n, lo, hi, stream);
}
int ogle_cuda_add(const float* a, const float* b, float* y, long n, ogle_stream_t stream) {
    return launch_elementwise<EW_ADD>(a, b, y, n, 0.f, 0.f, stream);
}

int ogle_cuda_add_act(const float* a, const float* b, float* y, long n, int act, float lo, float hi,
                      ogle_stream_t stream) {
    if (act == OGLE_ACT_NONE) return launch_elementwise<EW_ADD>(a, b, y, n, 0.f, 0.f, stream);
    if (act == OGLE_ACT_RELU) return launch_elementwise<EW_ADD_RELU>(a, b, y, n, 0.f, 0.f, stream);
    if (act == OGLE_ACT_CLIP) return launch_elementwise<EW_ADD_CLIP>(a, b, y, n, lo, hi, stream);
    return OGLE_ERR_INVALID;
}

int ogle_cuda_batchnorm(const float* x, const float* gamma, const float* beta, const float* mean,
                        const float* var, float* y, long pixels, int C, int channel_stride,
                        float eps, ogle_stream_t stream) {
    if (pixels < 0 || C <= 0) return OGLE_ERR_INVALID;
    if (channel_stride == 0) channel_stride = up4(C);
    if (channel_stride < C || (channel_stride & 3)) return OGLE_ERR_INVALID;
    if (pixels == 0) return OGLE_OK;
    if (!x || !y || !gamma || !beta || !mean || !var) return OGLE_ERR_INVALID;
    if (!aligned16(x) || !aligned16(y)) return OGLE_ERR_ALIGNMENT;
    const int q = channel_stride / 4;
    batchnorm_kernel<<<grid_for(pixels * q, 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(x), gamma, beta, mean, var, reinterpret_cast<float4*>(y),
        pixels, C, q, eps);
    return finish_launch();
}

}  // extern "C"

// Image front end of the detector (Detector::Preprocess,
// ogl_runtime/opengl/examples/ssd/detector.cc:99-109) on the device: an 8-bit BGR image
// becomes the network's float input in one pass - channel swap, bilinear resize with the
// 8-bit fixed-point arithmetic of OpenCV's default cv::resize (pixel-centre alignment, 11-bit
// weights, 32-bit row blend rounded to nearest; a horizontal tap outside the row becomes the
// edge pixel with weight 2048, a vertical tap outside the image keeps its fractional weights
// on the clamped row), conversion to float,
// mean subtraction - written straight into the padded NHWC4 layout. One thread per output
// pixel; the source is read through the read-only cache (each source pixel is used by at
// most four outputs when shrinking).
#include "common.cuh"

namespace ogle {
namespace {

struct Tap { int i0, i1, w0, w1; };

template <bool kClampWeights>
__device__ __forceinline__ Tap make_tap(int d, int dst, int src) {
    const double scale = src == dst ? 1.0 : double(src) / dst;     // frames already at the network's size skip the fp64 division
    float f = float((d + 0.5) * scale - 0.5);
    int s = int(floorf(f));
    f -= s;
    if (kClampWeights) {
        if (s < 0) { s = 0; f = 0.f; }
        if (s >= src - 1) { s = src - 1; f = 0.f; }
    }
    Tap t;
    t.i0 = min(max(s, 0), src - 1);
    t.i1 = min(max(s + 1, 0), src - 1);
    t.w0 = __float2int_rn((1.f - f) * 2048.f);
    t.w1 = __float2int_rn(f * 2048.f);
    return t;
}

__device__ __forceinline__ void preprocess_pixel(const unsigned char* __restrict__ src, int src_h, int src_w,
                                                 int src_row_bytes, float4* __restrict__ dst, int dst_h, int dst_w,
                                                 float3 mean, int x, int y) {
    const Tap tx = make_tap<true>(x, dst_w, src_w), ty = make_tap<false>(y, dst_h, src_h);
    const unsigned char* r0 = src + (size_t)ty.i0 * src_row_bytes;
    const unsigned char* r1 = src + (size_t)ty.i1 * src_row_bytes;
    float out[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const int sc = 2 - c;    // RGB channel c is BGR channel 2 - c
        const int h0 = __ldg(r0 + tx.i0 * 3 + sc) * tx.w0 + __ldg(r0 + tx.i1 * 3 + sc) * tx.w1;
        const int h1 = __ldg(r1 + tx.i0 * 3 + sc) * tx.w0 + __ldg(r1 + tx.i1 * 3 + sc) * tx.w1;
        int v = (((ty.w0 * (h0 >> 4)) >> 16) + ((ty.w1 * (h1 >> 4)) >> 16) + 2) >> 2;
        v = v < 0 ? 0 : (v > 255 ? 255 : v);
        out[c] = float(v);
    }
    dst[(size_t)y * dst_w + x] = make_float4(out[0] - mean.x, out[1] - mean.y, out[2] - mean.z, 0.f);
}

__global__ void preprocess_bgr8_kernel(const unsigned char* __restrict__ src, int src_h, int src_w, int src_row_bytes,
                                       float4* __restrict__ dst, int dst_h, int dst_w, float3 mean) {
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= dst_w || y >= dst_h) return;
    preprocess_pixel(src, src_h, src_w, src_row_bytes, dst, dst_h, dst_w, mean, x, y);
}

// A batch of images of any sizes in one launch: blockIdx.z walks the images, whose places in
// the byte buffer and sizes come from a table in device memory.
__global__ void preprocess_bgr8_batch_kernel(const unsigned char* __restrict__ base,
                                             const OgleImageDesc* __restrict__ descs, int n_images,
                                             float4* __restrict__ dst, int dst_h, int dst_w, float3 mean) {
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= dst_w || y >= dst_h) return;
    for (int i = blockIdx.z; i < n_images; i += gridDim.z) {
        const OgleImageDesc d = descs[i];
        preprocess_pixel(base + d.offset, d.height, d.width, d.row_bytes, dst + (size_t)i * dst_h * dst_w, dst_h, dst_w,
                         mean, x, y);
    }
}

}  // namespace
}  // namespace ogle

using namespace ogle;

extern "C" int ogle_cuda_preprocess_bgr8(const unsigned char* bgr, int src_h, int src_w, int src_row_bytes,
                                         float* dst_nhwc4, int dst_h, int dst_w, const float mean_rgb[3],
                                         ogle_stream_t stream) {
    if (!bgr || !dst_nhwc4 || !mean_rgb) return OGLE_ERR_INVALID;
    if (src_h <= 0 || src_w <= 0 || dst_h <= 0 || dst_w <= 0 || src_row_bytes < src_w * 3) return OGLE_ERR_INVALID;
    if (!aligned16(dst_nhwc4)) return OGLE_ERR_ALIGNMENT;
    const dim3 block(32, 8), grid(div_up(dst_w, 32), div_up(dst_h, 8));
    preprocess_bgr8_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
        bgr, src_h, src_w, src_row_bytes, reinterpret_cast<float4*>(dst_nhwc4), dst_h, dst_w,
        make_float3(mean_rgb[0], mean_rgb[1], mean_rgb[2]));
    return finish_launch();
}

extern "C" int ogle_cuda_preprocess_bgr8_batch(const unsigned char* base, const OgleImageDesc* descs_device, int n_images,
                                               float* dst_nhwc4, int dst_h, int dst_w, const float mean_rgb[3],
                                               ogle_stream_t stream) {
    if (n_images < 0 || dst_h <= 0 || dst_w <= 0 || !mean_rgb) return OGLE_ERR_INVALID;
    if (n_images == 0) return OGLE_OK;      // empty batch: nothing to read or write
    if (!base || !descs_device || !dst_nhwc4) return OGLE_ERR_INVALID;
    if (!aligned16(dst_nhwc4) || (reinterpret_cast<uintptr_t>(descs_device) & 7)) return OGLE_ERR_ALIGNMENT;
    const dim3 block(32, 8), grid(div_up(dst_w, 32), div_up(dst_h, 8), n_images < 65535 ? n_images : 65535);
    preprocess_bgr8_batch_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
        base, descs_device, n_images, reinterpret_cast<float4*>(dst_nhwc4), dst_h, dst_w,
        make_float3(mean_rgb[0], mean_rgb[1], mean_rgb[2]));
    return finish_launch();
}

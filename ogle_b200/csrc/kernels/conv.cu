// conv2d entry points: shape inference, filter packing and variant dispatch.
#include <cuda_bf16.h>

#include "conv_args.cuh"

namespace ogle {

int launch_conv_tc(const ConvArgs& a, int variant, int math_mode, const float* x,
                   const float* w_hi, const float* w_lo, const float* bias, float* y, cudaStream_t s,
                   float* y2 = nullptr, int K1 = 0, int split_col = 0, void* ws = nullptr, size_t ws_bytes = 0,
                   size_t* ws_needed = nullptr, const float* residual = nullptr, int res_ld = 0);
bool conv_tc_supported(const ConvArgs& a, int variant);
bool conv_tc_gather_supported(const ConvArgs& a, int variant);
bool dw_tma_supported(const ConvArgs& a);
bool conv_smallc_supported(const ConvArgs& a);

// Destination-indexed packing of an OIHW filter into the three sections of the
// packed blob (see FilterLayout).
__global__ void prepack_tap_major_kernel(const float* __restrict__ w, float* __restrict__ dst,
                                         int K, int Cg, int kernel, int Cp, int Kp) {
    const int taps = kernel * kernel;
    const long total = (long)taps * Cp * Kp;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int k = int(t % Kp); t /= Kp;
        const int c = int(t % Cp); t /= Cp;
        const int tap = int(t);
        float v = 0.f;
        if (k < K && c < Cg) v = w[((long)k * Cg + c) * taps + tap];
        dst[i] = v;
    }
}

__global__ void prepack_kmajor_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                      __nv_bfloat16* __restrict__ cross, int K, int Cg, int kernel,
                                      int Kp128, int Cp32) {
    const int taps = kernel * kernel;
    const long total = (long)Kp128 * taps * Cp32;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int c = int(t % Cp32); t /= Cp32;
        const int tap = int(t % taps); t /= taps;
        const int k = int(t);
        float v = 0.f;
        if (k < K && c < Cg) v = w[((long)k * Cg + c) * taps + tap];
        // hi keeps the 10 mantissa bits a TF32 operand carries; the cross section holds, per
        // 32-channel chunk, [bf16(w - hi) x 32 | bf16(w) x 32] for the BF16 pass
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        hi[i] = h;
        const long chunk = i - (c & 31);
        cross[chunk * 2 + (c & 31)] = __float2bfloat16_rn(v - h);
        cross[chunk * 2 + 32 + (c & 31)] = __float2bfloat16_rn(v);
    }
}

// Compact k-major sections for the gather form (see filter_compact): [Kp128][cols], column tap*Cg+c.
__global__ void prepack_kmajor_compact_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                              __nv_bfloat16* __restrict__ cross, int K, int Cg, int kernel, int cols,
                                              int Kp128) {
    const long total = (long)Kp128 * cols;
    const int taps = kernel * kernel;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int col = int(i % cols), k = int(i / cols);
        float v = 0.f;
        if (k < K && col < taps * Cg) {
            const int tap = col / Cg, c = col - tap * Cg;
            v = w[((long)k * Cg + c) * taps + tap];
        }
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        hi[i] = h;
        const int lane = col & 31;
        const long chunk = i - lane;         // first element of this 32-wide piece of the row
        cross[chunk * 2 + lane] = __float2bfloat16_rn(v - h);
        cross[chunk * 2 + 32 + lane] = __float2bfloat16_rn(v);
    }
}

static int fill_args(const OgleConvParams* p, ConvArgs* a, int* variant) {
    if (!p) return OGLE_ERR_INVALID;
    const int H = p->in_hwc[0], W = p->in_hwc[1], C = p->in_hwc[2];
    const int K = p->out_hwc[2];
    int group = p->group <= 0 ? 1 : p->group;   // conv2d.cc:91-94
    if (p->N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return OGLE_ERR_INVALID;
    if (p->kernel <= 0 || p->stride <= 0 || p->pad < 0 || p->dilation <= 0) return OGLE_ERR_INVALID;
    if (C % group || K % group) return OGLE_ERR_INVALID;
    if (p->act < 0 || p->act > 2) return OGLE_ERR_INVALID;
    const int eff = p->kernel * p->dilation - p->dilation + 1;   // conv2d.cc:191-194
    const int Ho = (H - eff + 2 * p->pad) / p->stride + 1;
    const int Wo = (W - eff + 2 * p->pad) / p->stride + 1;
    if (Ho <= 0 || Wo <= 0) return OGLE_ERR_INVALID;
    a->N = p->N; a->H = H; a->W = W; a->C = C;
    a->Cs = p->in_channel_stride ? p->in_channel_stride : up4(C);
    a->Ho = Ho; a->Wo = Wo; a->K = K;
    a->Ks = p->out_channel_stride ? p->out_channel_stride : up4(K);
    a->koff = p->out_channel_offset;
    if (a->Cs < up4(C) || (a->Cs & 3) || (a->Ks & 3) || (a->koff & 3) || a->koff < 0 ||
        a->koff + up4(K) > a->Ks)
        return OGLE_ERR_INVALID;
    a->kernel = p->kernel; a->stride = p->stride; a->pad = p->pad; a->dil = p->dilation; a->group = group;
    // shader choice, conv2d.cc:35-50
    if (p->kernel == 1 && group == 1 && p->dilation == 1 && p->stride == 1 && p->pad == 0) *variant = CONV_POINTWISE;
    else if (group != 1) *variant = (group == C && group == K) ? CONV_DEPTHWISE : CONV_GROUPED;
    else *variant = CONV_GENERAL;
    a->Cp = (*variant == CONV_DEPTHWISE) ? 1 : up4(C / group);
    a->Kp = up4(K);
    a->has_bias = p->has_bias ? 1 : 0;
    a->M = (long)p->N * Ho * Wo;
    if (p->n_tile < 0 || p->n_tile > 256 || (p->n_tile & 31)) return OGLE_ERR_INVALID;
    a->n_tile = p->n_tile;
    if (p->split < 0 || p->split > 16) return OGLE_ERR_INVALID;
    a->split = p->split;
    if (p->channels_on_m < 0 || p->channels_on_m > 2) return OGLE_ERR_INVALID;
    a->on_m = p->channels_on_m;
    if (p->sm_pair < 0 || p->sm_pair > 2) return OGLE_ERR_INVALID;
    a->pair = p->sm_pair;
    // activation, with the per-shader differences of the reference kept:
    //   pointwise clip clamps to [0, max] (conv2d_pw.glsl:85);
    //   grouped relu is max(min_value, v) (conv2d_grp.glsl:121).
    a->act = p->act; a->lo = p->min_value; a->hi = p->max_value;
    if (*variant == CONV_POINTWISE && p->act == OGLE_ACT_CLIP) a->lo = 0.f;
    if (*variant == CONV_GROUPED && p->act == OGLE_ACT_RELU) {
        a->act = OGLE_ACT_CLIP; a->lo = p->min_value; a->hi = __builtin_inff();
    }
    return OGLE_OK;
}

}  // namespace ogle

using namespace ogle;

extern "C" {

int ogle_cuda_conv2d_infer(OgleConvParams* p) {
    ConvArgs a; int variant;
    int rc = fill_args(p, &a, &variant);
    if (rc != OGLE_OK) return rc;
    p->out_hwc[0] = a.Ho; p->out_hwc[1] = a.Wo;
    return OGLE_OK;
}

size_t ogle_cuda_conv2d_filter_bytes(const OgleConvParams* p) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK) return 0;
    return filter_layout(a.K, a.C / a.group, a.kernel, a.group, a.Cp).total;
}

int ogle_cuda_conv2d_prepack(const OgleConvParams* p, const float* w_oihw, void* packed,
                             ogle_stream_t stream) {
    ConvArgs a; int variant;
    int rc = fill_args(p, &a, &variant);
    if (rc != OGLE_OK) return rc;
    if (!w_oihw || !packed) return OGLE_ERR_INVALID;
    if (!aligned16(packed)) return OGLE_ERR_ALIGNMENT;
    const int Cg = a.C / a.group;
    const FilterLayout L = filter_layout(a.K, Cg, a.kernel, a.group, a.Cp);
    cudaStream_t s = (cudaStream_t)stream;
    char* base = static_cast<char*>(packed);
    const long n0 = (long)a.kernel * a.kernel * a.Cp * a.Kp;
    prepack_tap_major_kernel<<<grid_for(n0, 256), 256, 0, s>>>(w_oihw, reinterpret_cast<float*>(base),
                                                               a.K, Cg, a.kernel, a.Cp, a.Kp);
    rc = finish_launch();
    if (rc != OGLE_OK) return rc;
    if (L.kmajor_bytes && filter_compact(Cg, a.kernel, a.group)) {
        const int cols = filter_compact_cols(Cg, a.kernel);
        prepack_kmajor_compact_kernel<<<grid_for((long)L.Kp128 * cols, 256), 256, 0, s>>>(
            w_oihw, reinterpret_cast<float*>(base + L.off_hi), reinterpret_cast<__nv_bfloat16*>(base + L.off_lo), a.K, Cg,
            a.kernel, cols, L.Kp128);
        rc = finish_launch();
    } else if (L.kmajor_bytes) {
        const long n1 = (long)L.Kp128 * a.kernel * a.kernel * L.Cp32;
        prepack_kmajor_kernel<<<grid_for(n1, 256), 256, 0, s>>>(
            w_oihw, reinterpret_cast<float*>(base + L.off_hi), reinterpret_cast<__nv_bfloat16*>(base + L.off_lo),
            a.K, Cg, a.kernel, L.Kp128, L.Cp32);
        rc = finish_launch();
    }
    return rc;
}

static bool served_by_tc(const OgleConvParams* p, const ConvArgs& a, int variant) {
    return p->math_mode != OGLE_MATH_FP32 && (variant == CONV_GENERAL || variant == CONV_POINTWISE) &&
           (conv_tc_supported(a, variant) || conv_tc_gather_supported(a, variant));
}

int ogle_cuda_conv2d_ws(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias, float* y,
                        void* workspace, size_t workspace_bytes, ogle_stream_t stream) {
    ConvArgs a; int variant;
    int rc = fill_args(p, &a, &variant);
    if (rc != OGLE_OK) return rc;
    if (a.Ho != p->out_hwc[0] || a.Wo != p->out_hwc[1]) return OGLE_ERR_INVALID;
    if (!x || !packed_filter || !y || (a.has_bias && !bias)) return OGLE_ERR_INVALID;
    if (!aligned16(x) || !aligned16(y) || !aligned16(packed_filter) || (workspace && !aligned16(workspace)))
        return OGLE_ERR_ALIGNMENT;
    if (p->math_mode < OGLE_MATH_FP32 || p->math_mode > OGLE_MATH_TF32X3) return OGLE_ERR_INVALID;
    const char* base = static_cast<const char*>(packed_filter);
    cudaStream_t s = (cudaStream_t)stream;
    if (served_by_tc(p, a, variant)) {
        const FilterLayout L = filter_layout(a.K, a.C / a.group, a.kernel, a.group, a.Cp);
        return launch_conv_tc(a, variant, p->math_mode, x, reinterpret_cast<const float*>(base + L.off_hi),
                              reinterpret_cast<const float*>(base + L.off_lo), bias, y, s, nullptr, 0, 0, workspace,
                              workspace ? workspace_bytes : 0);
    }
    return launch_conv_simt(a, variant, x, reinterpret_cast<const float*>(base), bias, y, s);
}

int ogle_cuda_conv2d_residual(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                              const float* residual, int residual_stride, float* y, ogle_stream_t stream) {
    ConvArgs a; int variant;
    int rc = fill_args(p, &a, &variant);
    if (rc != OGLE_OK) return rc;
    if (a.Ho != p->out_hwc[0] || a.Wo != p->out_hwc[1]) return OGLE_ERR_INVALID;
    if (!x || !packed_filter || !y || !residual || (a.has_bias && !bias)) return OGLE_ERR_INVALID;
    if (!aligned16(x) || !aligned16(y) || !aligned16(packed_filter) || !aligned16(residual)) return OGLE_ERR_ALIGNMENT;
    if (p->math_mode < OGLE_MATH_FP32 || p->math_mode > OGLE_MATH_TF32X3) return OGLE_ERR_INVALID;
    if (!ogle_cuda_conv2d_residual_supported(p)) return OGLE_ERR_UNSUPPORTED;
    const int ld = residual_stride ? residual_stride : a.Kp;
    if (ld < a.Kp || (ld & 3)) return OGLE_ERR_INVALID;
    const char* base = static_cast<const char*>(packed_filter);
    const FilterLayout L = filter_layout(a.K, a.C / a.group, a.kernel, a.group, a.Cp);
    return launch_conv_tc(a, variant, p->math_mode, x, reinterpret_cast<const float*>(base + L.off_hi),
                          reinterpret_cast<const float*>(base + L.off_lo), bias, y, (cudaStream_t)stream, nullptr, 0, 0, nullptr, 0,
                          nullptr, residual, ld);
}

int ogle_cuda_conv2d_residual_supported(const OgleConvParams* p) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK) return 0;
    return served_by_tc(p, a, variant) ? 1 : 0;
}

int ogle_cuda_conv2d(const OgleConvParams* p, const float* x, const void* packed_filter,
                     const float* bias, float* y, ogle_stream_t stream) {
    return ogle_cuda_conv2d_ws(p, x, packed_filter, bias, y, nullptr, 0, stream);
}

size_t ogle_cuda_conv2d_workspace_bytes(const OgleConvParams* p) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK || !served_by_tc(p, a, variant)) return 0;
    size_t need = 0;
    if (launch_conv_tc(a, variant, p->math_mode, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, 0,
                       &need) != OGLE_OK)
        return 0;
    return need;
}

const char* ogle_cuda_conv2d_kernel_name(const OgleConvParams* p) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK) return "";
    if (served_by_tc(p, a, variant)) return "conv_tc2_kernel";
    if (variant == CONV_DEPTHWISE) {
        if (dw_tma_supported(a)) return "dw3x3_tma_kernel";
        return (a.kernel == 3 && a.dil == 1 && (a.stride == 1 || a.stride == 2)) ? "dw3x3_kernel" : "dw_generic_kernel";
    }
    if (variant == CONV_GROUPED) return "grouped_kernel";
    if (variant == CONV_GENERAL && conv_smallc_supported(a)) return "conv3x3_smallc_kernel";
    return "conv_igemm_kernel";
}

int ogle_cuda_conv2d_pair_supported(const OgleConvParams* p) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK) return 0;
    if (p->math_mode == OGLE_MATH_FP32 || p->out_channel_stride || p->out_channel_offset) return 0;
    if (a.K > 256) return 0;                     // one N tile must hold both filters' columns
    return conv_tc_supported(a, variant) ? 1 : 0;
}

int ogle_cuda_conv2d_pair_ws(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                             int first_channels, int second_offset, float* y_first, float* y_second, void* workspace,
                             size_t workspace_bytes, ogle_stream_t stream) {
    ConvArgs a; int variant;
    int rc = fill_args(p, &a, &variant);
    if (rc != OGLE_OK) return rc;
    if (a.Ho != p->out_hwc[0] || a.Wo != p->out_hwc[1]) return OGLE_ERR_INVALID;
    if (!x || !packed_filter || !y_first || !y_second || (a.has_bias && !bias)) return OGLE_ERR_INVALID;
    if (!aligned16(x) || !aligned16(y_first) || !aligned16(y_second) || !aligned16(packed_filter) ||
        (workspace && !aligned16(workspace)))
        return OGLE_ERR_ALIGNMENT;
    if (first_channels <= 0 || second_offset != (first_channels + 31) / 32 * 32 || second_offset >= a.K)
        return OGLE_ERR_INVALID;
    if (!ogle_cuda_conv2d_pair_supported(p)) return OGLE_ERR_UNSUPPORTED;
    const char* base = static_cast<const char*>(packed_filter);
    const FilterLayout L = filter_layout(a.K, a.C / a.group, a.kernel, a.group, a.Cp);
    return launch_conv_tc(a, variant, p->math_mode, x, reinterpret_cast<const float*>(base + L.off_hi),
                          reinterpret_cast<const float*>(base + L.off_lo), bias, y_first, (cudaStream_t)stream,
                          y_second, first_channels, second_offset, workspace, workspace ? workspace_bytes : 0);
}

int ogle_cuda_conv2d_pair(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                          int first_channels, int second_offset, float* y_first, float* y_second,
                          ogle_stream_t stream) {
    return ogle_cuda_conv2d_pair_ws(p, x, packed_filter, bias, first_channels, second_offset, y_first, y_second, nullptr, 0,
                                    stream);
}

size_t ogle_cuda_conv2d_pair_workspace_bytes(const OgleConvParams* p, int first_channels, int second_offset) {
    ConvArgs a; int variant;
    if (fill_args(p, &a, &variant) != OGLE_OK || !ogle_cuda_conv2d_pair_supported(p)) return 0;
    if (first_channels <= 0 || second_offset != (first_channels + 31) / 32 * 32 || second_offset >= a.K) return 0;
    size_t need = 0;
    float dummy = 0.f;      // only its being non-null matters to the planner (two-output form)
    if (launch_conv_tc(a, variant, p->math_mode, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &dummy, first_channels,
                       second_offset, nullptr, 0, &need) != OGLE_OK)
        return 0;
    return need;
}

}  // extern "C"

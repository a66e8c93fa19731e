// Test infrastructure only. Builds oracle/_ref/libogle_ref.so from the
// reference's OWN sources, read where they lie (never copied):
//   - the fragment shaders under ogl_runtime/opengl/nn/glsl/, compiled verbatim
//     as C++ through oracle/glsl_shim.h, one namespace per shader and per
//     build-option combination;
//   - ogl_runtime/opengl/core/cpu_functor.cc (layout converters and the CPU box
//     decoder), compiled unmodified against oracle/ref_shim/ headers.
// This file only drives them: it pads inputs with the reference's converters,
// sets the uniforms that the matching Kernel::Compute sets, runs main() once per
// output texel, and unpads. It exports the interface in oracle/oracle.h.
//
// The whole library is compiled with -ftrivial-auto-var-init=zero because
// gemm.glsl:28 accumulates into an uninitialised float[4]; GL implementations
// give zero there in practice, and that flag gives the same in C++.
#include <vector>
#include <cstring>
#include <omp.h>
#include "glsl_shim.h"
#include "oracle.h"
#include "opengl/core/tensor.h"       // oracle/ref_shim version
#include "opengl/core/cpu_functor.h"  // the reference's own header

#undef UP_DIV    // the shaders define their own
#undef UP_ROUND

using namespace glsl;
static thread_local FragCoord gl_FragCoord;
static const int kMaxTex = 268435456;  // == MAX_TEXTURE_SIZE of glsl_keywords.h

namespace {

template <class F>
void run_grid(float* out, long grid_w, long grid_h, F frag) {
    const long total = grid_w * grid_h;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < total; ++i) {
        const long x = i % grid_w, y = i / grid_w;
        gl_FragCoord.xy.x = float(x) + 0.5f;
        gl_FragCoord.xy.y = float(y) + 0.5f;
        const vec4 c = frag();
        float* o = out + i * 4;
        o[0] = c.x; o[1] = c.y; o[2] = c.z; o[3] = c.w;
    }
}

struct ConvCall {
    sampler2D image, filter, bias;
    int stride, kernel, group, dilation, pad, use_bias, act;
    float minv, maxv;
    int H, W, C, Ho, Wo, K, N;
    float* dst;
};

inline int up4(int v) { return (v + 3) / 4 * 4; }
inline int div4(int v) { return (v + 3) / 4; }

// Pads the last dimension to a multiple of 4 with the reference's converter.
std::vector<float> pad_last(const float* x, long rows, int last) {
    std::vector<float> dst(size_t(rows) * up4(last));
    opengl::Tensor s(const_cast<float*>(x), {int(rows), last}, size_t(rows) * last);
    opengl::Tensor d(dst.data(), {int(rows), last}, dst.size());
    opengl::host_functor::ConvertTensorANYToANY4()(nullptr, &s, &d);
    return dst;
}
void unpad_last(const std::vector<float>& x4, float* y, long rows, int last) {
    opengl::Tensor s(const_cast<float*>(x4.data()), {int(rows), last}, x4.size());
    opengl::Tensor d(y, {int(rows), last}, size_t(rows) * last);
    opengl::host_functor::ConvertTensorANY4ToANY()(nullptr, &s, &d);
}

}  // namespace

#define REF_DEFINE_CONV_RUNNER(fn, NS)                                              \
    static void fn(const ConvCall& c) {                                             \
        NS::input_image = c.image; NS::input_filter = c.filter; NS::input_bias = c.bias; \
        NS::stride_size = c.stride; NS::kernel_size = c.kernel; NS::group = c.group; \
        NS::dilation = c.dilation; NS::padding = c.pad; NS::use_bias = c.use_bias;  \
        NS::act = c.act; NS::min_value = c.minv; NS::max_value = c.maxv;            \
        NS::input_shape = ivec3{c.H, c.W, c.C};                                     \
        NS::output_shape = ivec3{c.Ho, c.Wo, c.K};                                  \
        run_grid(c.dst, long(c.Wo) * div4(c.K), long(c.N) * c.Ho,                   \
                 []() { NS::main(); return NS::color; });                           \
    }

#include "glsl_keywords.h"  // from here on `out` and `uniform` are GLSL qualifiers

// bias x activation build-option combinations
#define REF_VARIANT_NS conv_b0_a0
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS

#define USE_CLIP
#define REF_VARIANT_NS conv_b0_a1
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS
#undef USE_CLIP

#define USE_RELU
#define REF_VARIANT_NS conv_b0_a2
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS
#undef USE_RELU

#define USE_BIAS
#define REF_VARIANT_NS conv_b1_a0
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS

#define USE_CLIP
#define REF_VARIANT_NS conv_b1_a1
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS
#undef USE_CLIP

#define USE_RELU
#define REF_VARIANT_NS conv_b1_a2
#include "ref_conv_variants.inc"
#undef REF_VARIANT_NS
#undef USE_RELU
#undef USE_BIAS

namespace sh_pool {
#include "opengl/nn/glsl/pool.glsl"
}
namespace sh_bn {
#include "opengl/nn/glsl/batchnorm.glsl"
}
namespace sh_relu {
#include "opengl/nn/glsl/relu.glsl"
}
namespace sh_clip {
#include "opengl/nn/glsl/clip.glsl"
}
namespace sh_add {
#include "opengl/nn/glsl/binary.glsl"
}
namespace sh_gemm {
#include "opengl/nn/glsl/gemm.glsl"
}
namespace sh_concat {
#include "opengl/nn/glsl/concat_multi.glsl"
}
namespace sh_transpose {
#include "opengl/nn/glsl/transpose_any4.glsl"
}

#undef out
#undef uniform

namespace {
typedef void (*ConvRunner)(const ConvCall&);
// [variant][bias][act]; variant: 0 general, 1 pointwise, 2 depthwise, 3 grouped
const ConvRunner kConvRunners[4][2][3] = {
    {{conv_b0_a0::run_general, conv_b0_a1::run_general, conv_b0_a2::run_general},
     {conv_b1_a0::run_general, conv_b1_a1::run_general, conv_b1_a2::run_general}},
    {{conv_b0_a0::run_pw, conv_b0_a1::run_pw, conv_b0_a2::run_pw},
     {conv_b1_a0::run_pw, conv_b1_a1::run_pw, conv_b1_a2::run_pw}},
    {{conv_b0_a0::run_dw, conv_b0_a1::run_dw, conv_b0_a2::run_dw},
     {conv_b1_a0::run_dw, conv_b1_a1::run_dw, conv_b1_a2::run_dw}},
    {{conv_b0_a0::run_grp, conv_b0_a1::run_grp, conv_b0_a2::run_grp},
     {conv_b1_a0::run_grp, conv_b1_a1::run_grp, conv_b1_a2::run_grp}},
};
}  // namespace

extern "C" {

int ogle_oracle_threads(void) { return omp_get_max_threads(); }
void ogle_oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

int ogle_oracle_conv2d(const float* x, const float* w, const float* bias, float* y,
                       int N, int H, int W, int C, int K, int kernel, int stride, int pad,
                       int dilation, int group, int act, float minv, float maxv) {
    if (group <= 0) group = 1;
    if (C % group || K % group || act < 0 || act > 2) return -1;
    const int eff = kernel * dilation - dilation + 1;
    const int Ho = (H - eff + 2 * pad) / stride + 1;
    const int Wo = (W - eff + 2 * pad) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return -1;
    // shader choice, conv2d.cc:35-50
    int variant;
    if (kernel == 1 && group == 1 && dilation == 1 && stride == 1 && pad == 0) variant = 1;
    else if (group != 1) variant = (group == C && group == K) ? 2 : 3;
    else variant = 0;

    const int Cg = C / group;
    std::vector<float> x4 = pad_last(x, long(N) * H * W, C);
    // filter: reference NCHW -> HWN4C4 converter, cpu_functor.cc:87-116
    std::vector<float> f4(size_t(kernel) * kernel * div4(K) * up4(Cg) * 4);
    {
        opengl::Tensor s(const_cast<float*>(w), {K, Cg, kernel, kernel}, size_t(K) * Cg * kernel * kernel);
        opengl::Tensor d(f4.data(), {K, Cg, kernel, kernel}, f4.size());
        opengl::host_functor::ConvertTensorNCHWToHWN4C4()(nullptr, &s, &d);
    }
    std::vector<float> b4;
    if (bias) b4 = pad_last(bias, 1, K);
    std::vector<float> y4(size_t(N) * Ho * Wo * up4(K));

    ConvCall c;
    c.image = sampler2D{x4.data(), W * div4(C), N * H};
    c.filter = sampler2D{f4.data(), up4(Cg), kernel * kernel * div4(K)};
    c.bias = sampler2D{bias ? b4.data() : nullptr, kMaxTex, 1};
    c.stride = stride; c.kernel = kernel; c.group = group; c.dilation = dilation; c.pad = pad;
    c.use_bias = bias ? 1 : 0; c.act = act; c.minv = minv; c.maxv = maxv;
    c.H = H; c.W = W; c.C = C; c.Ho = Ho; c.Wo = Wo; c.K = K; c.N = N;
    c.dst = y4.data();
    kConvRunners[variant][bias ? 1 : 0][act](c);
    unpad_last(y4, y, long(N) * Ho * Wo, K);
    return 0;
}

int ogle_oracle_pool(const float* x, float* y, int N, int H, int W, int C,
                     int kernel, int stride, int pad, int type) {
    const int Ho = (H - kernel + 2 * pad) / stride + 1;
    const int Wo = (W - kernel + 2 * pad) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return -1;
    std::vector<float> x4 = pad_last(x, long(N) * H * W, C);
    std::vector<float> y4(size_t(N) * Ho * Wo * up4(C));
    sh_pool::input_image = sampler2D{x4.data(), W * div4(C), N * H};
    sh_pool::kernel_size = kernel; sh_pool::stride_size = stride; sh_pool::padding = pad;
    sh_pool::pool_type = type;
    sh_pool::input_shape = ivec3{H, W, C};
    sh_pool::output_shape = ivec3{Ho, Wo, C};
    run_grid(y4.data(), long(Wo) * div4(C), long(N) * Ho, []() { sh_pool::main(); return sh_pool::color; });
    unpad_last(y4, y, long(N) * Ho * Wo, C);
    return 0;
}

int ogle_oracle_batchnorm(const float* x, const float* gamma, const float* beta,
                          const float* mean, const float* var, float* y,
                          int N, int H, int W, int C, float eps) {
    std::vector<float> x4 = pad_last(x, long(N) * H * W, C);
    std::vector<float> g4 = pad_last(gamma, 1, C), b4 = pad_last(beta, 1, C);
    std::vector<float> m4 = pad_last(mean, 1, C), v4 = pad_last(var, 1, C);
    // padded variance lanes are 0; with eps > 0 they stay finite and are dropped on unpad
    std::vector<float> y4(x4.size());
    sh_bn::input_image = sampler2D{x4.data(), W * div4(C), N * H};
    sh_bn::input_gamma = sampler2D{g4.data(), div4(C), 1};
    sh_bn::input_beta = sampler2D{b4.data(), div4(C), 1};
    sh_bn::input_mean = sampler2D{m4.data(), div4(C), 1};
    sh_bn::input_var = sampler2D{v4.data(), div4(C), 1};
    sh_bn::momentum = 0.f; sh_bn::eps = eps;
    sh_bn::output_shape = ivec3{H, W, C};
    run_grid(y4.data(), long(W) * div4(C), long(N) * H, []() { sh_bn::main(); return sh_bn::color; });
    unpad_last(y4, y, long(N) * H * W, C);
    return 0;
}

// Elementwise shaders see the tensor as texels; n is padded up to a multiple of 4 here.
static std::vector<float> as_texels(const float* x, long n) {
    std::vector<float> t(size_t((n + 3) / 4 * 4), 0.f);
    std::memcpy(t.data(), x, size_t(n) * sizeof(float));
    return t;
}

int ogle_oracle_relu(const float* x, float* y, long n) {
    std::vector<float> t = as_texels(x, n), o(t.size());
    sh_relu::input_image = sampler2D{t.data(), int(t.size() / 4), 1};
    run_grid(o.data(), long(t.size() / 4), 1, []() { sh_relu::main(); return sh_relu::color; });
    std::memcpy(y, o.data(), size_t(n) * sizeof(float));
    return 0;
}

int ogle_oracle_clip(const float* x, float* y, long n, float lo, float hi) {
    std::vector<float> t = as_texels(x, n), o(t.size());
    sh_clip::input_image = sampler2D{t.data(), int(t.size() / 4), 1};
    sh_clip::min_value = lo; sh_clip::max_value = hi;
    run_grid(o.data(), long(t.size() / 4), 1, []() { sh_clip::main(); return sh_clip::color; });
    std::memcpy(y, o.data(), size_t(n) * sizeof(float));
    return 0;
}

int ogle_oracle_add(const float* a, const float* b, float* y, long n) {
    std::vector<float> ta = as_texels(a, n), tb = as_texels(b, n), o(ta.size());
    sh_add::input0 = sampler2D{ta.data(), int(ta.size() / 4), 1};
    sh_add::input1 = sampler2D{tb.data(), int(tb.size() / 4), 1};
    run_grid(o.data(), long(ta.size() / 4), 1, []() { sh_add::main(); return sh_add::color; });
    std::memcpy(y, o.data(), size_t(n) * sizeof(float));
    return 0;
}

int ogle_oracle_gemm(const float* A, const float* B, const float* C, float* Y,
                     int M, int K, int N, int transB, float alpha, float beta, int bias_mode) {
    // The shader reads C at the output's own texel (gemm.glsl:92-94): defined for
    // C of shape [M,N], or [N] when M == 1. Anything else is outside the reference.
    if (bias_mode == 2 && M != 1) return -2;
    std::vector<float> a4 = pad_last(A, M, K);
    std::vector<float> b4 = transB ? pad_last(B, N, K) : pad_last(B, K, N);
    std::vector<float> c4;
    if (bias_mode) c4 = pad_last(C, bias_mode == 1 ? M : 1, N);
    std::vector<float> y4(size_t(M) * up4(N));
    sh_gemm::A = sampler2D{a4.data(), kMaxTex, 1};
    sh_gemm::B = sampler2D{b4.data(), kMaxTex, 1};
    sh_gemm::C = sampler2D{bias_mode ? c4.data() : nullptr, kMaxTex, 1};
    sh_gemm::alpha = alpha; sh_gemm::beta = beta;
    sh_gemm::use_bias = bias_mode ? 1 : 0; sh_gemm::transb = transB;
    sh_gemm::input_shape = ivec2(M, K);
    sh_gemm::output_shape = ivec2(M, N);
    run_grid(y4.data(), long(M) * div4(N), 1, []() { sh_gemm::main(); return sh_gemm::color; });
    unpad_last(y4, Y, M, N);
    return 0;
}

int ogle_oracle_concat(int n_inputs, const float* const* xs, const int* in_shapes4,
                       int axis, float* y) {
    if (axis < 0 || axis > 3 || n_inputs < 1) return -1;
    int os[4] = {in_shapes4[0], in_shapes4[1], in_shapes4[2], in_shapes4[3]};
    os[axis] = 0;
    for (int i = 0; i < n_inputs; ++i) os[axis] += in_shapes4[i * 4 + axis];
    const long orows = long(os[0]) * os[1] * os[2];
    std::vector<float> y4(size_t(orows) * up4(os[3]), 0.f);
    sh_concat::output_shape = ivec4{os[0], os[1], os[2], os[3]};
    sh_concat::axis = axis;
    int axis_offset = 0;
    for (int i = 0; i < n_inputs; ++i) {
        const int* s = in_shapes4 + i * 4;
        std::vector<float> x4 = pad_last(xs[i], long(s[0]) * s[1] * s[2], s[3]);
        sh_concat::input_image = sampler2D{x4.data(), kMaxTex, 1};
        sh_concat::origin_image = sampler2D{y4.data(), kMaxTex, 1};
        sh_concat::input_shape = ivec4{s[0], s[1], s[2], s[3]};
        sh_concat::axis_offset = axis_offset;
        // each fragment reads the output only at its own position, so the
        // read-while-write of concat.cc:73-96 is safe in place
        run_grid(y4.data(), orows * div4(os[3]), 1, []() { sh_concat::main(); return sh_concat::color; });
        axis_offset += s[axis];
    }
    unpad_last(y4, y, orows, os[3]);
    return 0;
}

int ogle_oracle_transpose(const float* x, const int* is, const int* perm, float* y) {
    int os[4];
    for (int i = 0; i < 4; ++i) os[i] = is[perm[i]];
    std::vector<float> x4 = pad_last(x, long(is[0]) * is[1] * is[2], is[3]);
    const long orows = long(os[0]) * os[1] * os[2];
    std::vector<float> y4(size_t(orows) * up4(os[3]));
    sh_transpose::input_image = sampler2D{x4.data(), kMaxTex, 1};
    sh_transpose::perm = ivec4{perm[0], perm[1], perm[2], perm[3]};
    sh_transpose::input_shape = ivec4{is[0], is[1], is[2], is[3]};
    sh_transpose::output_shape = ivec4{os[0], os[1], os[2], os[3]};
    run_grid(y4.data(), orows * div4(os[3]), 1, []() { sh_transpose::main(); return sh_transpose::color; });
    unpad_last(y4, y, orows, os[3]);
    return 0;
}

int ogle_oracle_decode(const float* pred, const float* anchors, float* out,
                       int N, int A, const float* variances4) {
    // The reference defines one image per call (anchors are read at the
    // prediction's own index); images are decoded one at a time here.
    std::vector<float> var(variances4, variances4 + 4);
    for (int n = 0; n < N; ++n) {
        opengl::Tensor p(const_cast<float*>(pred) + size_t(n) * A * 4, {1, A, 4}, size_t(A) * 4);
        opengl::Tensor a(const_cast<float*>(anchors), {A, 4}, size_t(A) * 4);
        opengl::Tensor d(out + size_t(n) * A * 4, {1, A, 4}, size_t(A) * 4);
        opengl::host_functor::SSDBBoxDecoder()(nullptr, &p, &a, &d, var);
    }
    return 0;
}

int ogle_oracle_pad4(const float* x, float* y, long rows, int last) {
    std::vector<float> t = pad_last(x, rows, last);
    std::memcpy(y, t.data(), t.size() * sizeof(float));
    return 0;
}

int ogle_oracle_unpad4(const float* x, float* y, long rows, int last) {
    std::vector<float> t(x, x + size_t(rows) * up4(last));
    unpad_last(t, y, rows, last);
    return 0;
}

int ogle_oracle_prepack_filter(const float* w, float* packed, int O, int I, int kh, int kw) {
    const size_t n = size_t(kh) * kw * div4(O) * up4(I) * 4;
    opengl::Tensor s(const_cast<float*>(w), {O, I, kh, kw}, size_t(O) * I * kh * kw);
    opengl::Tensor d(packed, {O, I, kh, kw}, n);
    opengl::host_functor::ConvertTensorNCHWToHWN4C4()(nullptr, &s, &d);
    return 0;
}

int ogle_oracle_unpack_filter(const float* packed, float* w, int O, int I, int kh, int kw) {
    const size_t n = size_t(kh) * kw * div4(O) * up4(I) * 4;
    opengl::Tensor s(const_cast<float*>(packed), {O, I, kh, kw}, n);
    opengl::Tensor d(w, {O, I, kh, kw}, size_t(O) * I * kh * kw);
    opengl::host_functor::ConvertTensorHWN4C4ToNCHW()(nullptr, &s, &d);
    return 0;
}

// The Detector post-process needs OpenCV types in the reference; not built here.
int ogle_oracle_detect(const float*, const float*, int, int, int, int, float, int, float,
                       int*, float*, int*, int*) { return -100; }
int ogle_oracle_topk_per_class(const float*, int, int, float, int, float*, int*, int*) { return -100; }
int ogle_oracle_preprocess_bgr8(const unsigned char*, int, int, int, float*, int, int, const float*) { return -100; }

}  // extern "C"

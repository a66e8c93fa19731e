// Test infrastructure only. CPU restatement of the arithmetic on the OGLE hot
// path, in the reference's evaluation order, exporting oracle/oracle.h.
// Only tests, the smoke check and the benchmark's CPU-baseline leg may load it;
// the product library never does.
//
// Pinning: the reference holds no golden vectors for this path; every function
// below is checked bit for bit (tests/test_oracle.py) against
// oracle/_ref/libogle_ref.so, which is the reference's own shader, functor and
// detector source compiled for the CPU, and against that library's outputs
// committed under tests/golden/. ogle_oracle_detect is pinned against the
// reference's Detector::GenerateBoxInfo / GetTopK / NMS; ogle_oracle_preprocess_bgr8
// against OpenCV (cv2). ogle_oracle_topk_per_class is an extension the reference
// does not contain: its softmax is pinned against the reference's, its selection
// rule (threshold, order by score then anchor, first k) has no counterpart to pin to.
//
// Device layouts of the reference, restated:
//   NHWC4 / ANY4 : last dimension padded with zeros to a multiple of 4;
//   HWN4C4       : filter OIHW -> [(kh*kw)*ceil(O/4)] rows x [ceil(I/4)*4] texels
//                  x 4 output lanes.
// In the shaders one fragment computes one texel = 4 consecutive output
// channels; the padded input lanes take part in the sums (as zeros), which
// matters for bit-exactness and is reproduced here.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>
#include <omp.h>
#include "oracle.h"

namespace {

inline int up4(int v) { return (v + 3) / 4 * 4; }
inline int div4(int v) { return (v + 3) / 4; }

// ANY -> ANY4, ogl_runtime/opengl/core/cpu_functor.cc:10-27
std::vector<float> pad_last(const float* x, long rows, int last) {
    const int l4 = up4(last);
    std::vector<float> d(size_t(rows) * l4, 0.f);
    for (long r = 0; r < rows; ++r)
        std::memcpy(&d[size_t(r) * l4], x + size_t(r) * last, size_t(last) * sizeof(float));
    return d;
}

// One 4x4 block times one texel, summed left to right:
// mat4(k0,k1,k2,k3) * v = ((k0*v.x + k1*v.y) + k2*v.z) + k3*v.w
inline float mat_row(const float* k0, const float* k1, const float* k2, const float* k3,
                     int lane, const float* v) {
    return ((k0[lane] * v[0] + k1[lane] * v[1]) + k2[lane] * v[2]) + k3[lane] * v[3];
}

inline float activate(float v, int act, float lo, float hi) {
    // conv2d.glsl:82-90: clamp = min(max(v,lo),hi); relu = max(0,v)
    if (act == 1) return std::min(std::max(v, lo), hi);
    if (act == 2) return std::max(0.f, v);
    return v;
}

}  // namespace

extern "C" {

int ogle_oracle_threads(void) { return omp_get_max_threads(); }
void ogle_oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

int ogle_oracle_prepack_filter(const float* w, float* packed, int O, int I, int kh, int kw) {
    // ogl_runtime/opengl/core/cpu_functor.cc:87-116
    const int i4 = div4(I), o4 = div4(O);
    std::memset(packed, 0, size_t(kh) * kw * o4 * i4 * 4 * 4 * sizeof(float));
    for (int o = 0; o < O; ++o)
        for (int i = 0; i < I; ++i)
            for (int h = 0; h < kh; ++h)
                for (int x = 0; x < kw; ++x) {
                    const size_t row = size_t(h * kw + x) * o4 + o / 4;
                    const size_t texel = row * (size_t(i4) * 4) + size_t(i / 4) * 4 + i % 4;
                    packed[texel * 4 + o % 4] = w[((size_t(o) * I + i) * kh + h) * kw + x];
                }
    return 0;
}

int ogle_oracle_unpack_filter(const float* packed, float* w, int O, int I, int kh, int kw) {
    // ogl_runtime/opengl/core/cpu_functor.cc:55-85
    const int i4 = div4(I), o4 = div4(O);
    for (int o = 0; o < O; ++o)
        for (int i = 0; i < I; ++i)
            for (int h = 0; h < kh; ++h)
                for (int x = 0; x < kw; ++x) {
                    const size_t row = size_t(h * kw + x) * o4 + o / 4;
                    const size_t texel = row * (size_t(i4) * 4) + size_t(i / 4) * 4 + i % 4;
                    w[((size_t(o) * I + i) * kh + h) * kw + x] = packed[texel * 4 + o % 4];
                }
    return 0;
}

int ogle_oracle_pad4(const float* x, float* y, long rows, int last) {
    std::vector<float> t = pad_last(x, rows, last);
    std::memcpy(y, t.data(), t.size() * sizeof(float));
    return 0;
}

int ogle_oracle_unpad4(const float* x, float* y, long rows, int last) {
    // ogl_runtime/opengl/core/cpu_functor.cc:29-47
    const int l4 = up4(last);
    for (long r = 0; r < rows; ++r)
        std::memcpy(y + size_t(r) * last, x + size_t(r) * l4, size_t(last) * sizeof(float));
    return 0;
}

int ogle_oracle_conv2d(const float* x, const float* w, const float* bias, float* y,
                       int N, int H, int W, int C, int K, int kernel, int stride, int pad,
                       int dilation, int group, int act, float lo, float hi) {
    if (group <= 0) group = 1;  // conv2d.cc:91-94
    if (C % group || K % group || act < 0 || act > 2) return -1;
    const int eff = kernel * dilation - dilation + 1;  // conv2d.cc:191-194
    const int Ho = (H - eff + 2 * pad) / stride + 1;
    const int Wo = (W - eff + 2 * pad) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return -1;
    const bool pointwise = kernel == 1 && group == 1 && dilation == 1 && stride == 1 && pad == 0;
    const bool depthwise = !pointwise && group != 1 && group == C && group == K;
    const bool grouped = !pointwise && group != 1 && !depthwise;
    const int Cg = C / group, Kg = K / group;
    const int C4 = div4(C), K4 = div4(K), Cg4 = div4(Cg);

    std::vector<float> x4 = pad_last(x, long(N) * H * W, C);
    std::vector<float> f4(size_t(kernel) * kernel * K4 * Cg4 * 16);
    ogle_oracle_prepack_filter(w, f4.data(), K, Cg, kernel, kernel);
    const size_t frow = size_t(Cg4) * 16;  // floats per filter-texture row

#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int oy = 0; oy < Ho; ++oy)
            for (int ox = 0; ox < Wo; ++ox)
                for (int k4 = 0; k4 < K4; ++k4) {
                    float acc[4];
                    for (int l = 0; l < 4; ++l) {
                        const int k = k4 * 4 + l;
                        acc[l] = (bias && k < K) ? bias[k] : 0.f;
                    }
                    if (grouped) {
                        // conv2d_grp.glsl:50-109: scalar sum per lane, x (i) outer, y (j)
                        // inner, starting from 0 and added to the bias at the end
                        for (int l = 0; l < 4; ++l) {
                            const int k = k4 * 4 + l;
                            const int g = k / Kg;  // lanes past K read zero filter texels
                            float v = 0.f;
                            for (int i = 0; i < kernel; ++i)
                                for (int j = 0; j < kernel; ++j) {
                                    const int ix = ox * stride + i * dilation - pad;
                                    const int iy = oy * stride + j * dilation - pad;
                                    if (ix < 0 || ix >= W || iy < 0 || iy >= H) continue;
                                    for (int c = 0; c < Cg; ++c) {
                                        const int ci = c + g * Cg;
                                        // for padded lanes (k >= K) g may point past the last
                                        // group; the filter value is 0 there, and the image
                                        // texel fetch is out of range in the reference too
                                        if (k >= K) continue;
                                        const float a = x4[((size_t(n) * H + iy) * W + ix) * (C4 * 4) + ci];
                                        const size_t row = size_t(j * kernel + i) * K4 + k / 4;
                                        const float b = f4[row * frow + size_t(c) * 4 + k % 4];
                                        v += a * b;
                                    }
                                }
                            acc[l] += v;
                        }
                    } else if (depthwise) {
                        // conv2d_dw.glsl:64-85: per tap, acc += k_texel * in_texel
                        for (int j = 0; j < kernel; ++j)
                            for (int i = 0; i < kernel; ++i) {
                                const int ix = i * dilation + ox * stride - pad;
                                const int iy = j * dilation + oy * stride - pad;
                                if (ix < 0 || ix >= W || iy < 0 || iy >= H) continue;
                                const float* v = &x4[((size_t(n) * H + iy) * W + ix) * (C4 * 4) + k4 * 4];
                                const float* f = &f4[(size_t(j * kernel + i) * K4 + k4) * frow];
                                for (int l = 0; l < 4; ++l) acc[l] += f[l] * v[l];
                            }
                    } else {
                        // conv2d.glsl:47-80 and conv2d_pw.glsl:57-80:
                        // rows (j) outer, columns (i) inner, then input texels
                        for (int j = 0; j < kernel; ++j)
                            for (int i = 0; i < kernel; ++i) {
                                const int ix = ox * stride + i * dilation - pad;
                                const int iy = oy * stride + j * dilation - pad;
                                if (ix < 0 || ix >= W || iy < 0 || iy >= H) continue;
                                const float* px = &x4[((size_t(n) * H + iy) * W + ix) * (C4 * 4)];
                                const float* f = &f4[(size_t(j * kernel + i) * K4 + k4) * frow];
                                for (int c4 = 0; c4 < C4; ++c4) {
                                    const float* kt = f + size_t(c4) * 16;
                                    const float* v = px + c4 * 4;
                                    for (int l = 0; l < 4; ++l)
                                        acc[l] += mat_row(kt, kt + 4, kt + 8, kt + 12, l, v);
                                }
                            }
                    }
                    for (int l = 0; l < 4; ++l) {
                        const int k = k4 * 4 + l;
                        if (k >= K) continue;
                        float v = acc[l];
                        if (pointwise && act == 1) v = std::min(std::max(v, 0.f), hi);  // conv2d_pw.glsl:85
                        else if (grouped && act == 1) v = std::min(hi, std::max(lo, v));  // conv2d_grp.glsl:114-117
                        else if (grouped && act == 2) v = std::max(lo, v);                // conv2d_grp.glsl:121
                        else v = activate(v, act, lo, hi);
                        y[((size_t(n) * Ho + oy) * Wo + ox) * K + k] = v;
                    }
                }
    return 0;
}

int ogle_oracle_pool(const float* x, float* y, int N, int H, int W, int C,
                     int kernel, int stride, int pad, int type) {
    const int Ho = (H - kernel + 2 * pad) / stride + 1;  // pool.cc:104-107
    const int Wo = (W - kernel + 2 * pad) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return -1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int oy = 0; oy < Ho; ++oy)
            for (int ox = 0; ox < Wo; ++ox)
                for (int c = 0; c < C; ++c) {
                    // pool.glsl:27-65: columns (i) outer, rows (j) inner
                    bool first = true;
                    float v = 0.f;
                    for (int i = 0; i < kernel; ++i)
                        for (int j = 0; j < kernel; ++j) {
                            const int ix = ox * stride + i - pad;
                            const int iy = oy * stride + j - pad;
                            if (ix < 0 || ix >= W || iy < 0 || iy >= H) continue;
                            const float item = x[((size_t(n) * H + iy) * W + ix) * C + c];
                            if (type == 0) {
                                if (first) { v = item; first = false; }
                                else v = std::max(v, item);
                            } else {
                                v += item;
                            }
                        }
                    if (type != 0) v = v / float(kernel * kernel);
                    y[((size_t(n) * Ho + oy) * Wo + ox) * C + c] = v;
                }
    return 0;
}

int ogle_oracle_batchnorm(const float* x, const float* gamma, const float* beta,
                          const float* mean, const float* var, float* y,
                          int N, int H, int W, int C, float eps) {
    const long rows = long(N) * H * W;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (int c = 0; c < C; ++c)  // batchnorm.glsl:31
            y[r * C + c] = (x[r * C + c] - mean[c]) / std::sqrt(var[c] + eps) * gamma[c] + beta[c];
    return 0;
}

int ogle_oracle_relu(const float* x, float* y, long n) {
    for (long i = 0; i < n; ++i) y[i] = std::max(0.f, x[i]);
    return 0;
}
int ogle_oracle_clip(const float* x, float* y, long n, float lo, float hi) {
    for (long i = 0; i < n; ++i) y[i] = std::min(hi, std::max(lo, x[i]));  // clip.glsl:8-9
    return 0;
}
int ogle_oracle_add(const float* a, const float* b, float* y, long n) {
    for (long i = 0; i < n; ++i) y[i] = a[i] + b[i];
    return 0;
}

int ogle_oracle_gemm(const float* A, const float* B, const float* C, float* Y,
                     int M, int K, int N, int transB, float alpha, float beta, int bias_mode) {
    // gemm.glsl:36-94: res starts at 0, res += alpha*a*b (left to right) over k,
    // then + beta*C. Row-broadcast of a [N] bias for M > 1 is the ONNX meaning;
    // the reference itself only defines it for M == 1.
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float res = 0.f;
            for (int m = 0; m < K; ++m) {
                const float a = A[size_t(i) * K + m];
                const float b = transB ? B[size_t(j) * K + m] : B[size_t(m) * N + j];
                res += alpha * a * b;
            }
            if (bias_mode == 1) res += beta * C[size_t(i) * N + j];
            else if (bias_mode == 2) res += beta * C[j];
            Y[size_t(i) * N + j] = res;
        }
    return 0;
}

int ogle_oracle_concat(int n_inputs, const float* const* xs, const int* in_shapes4,
                       int axis, float* y) {
    if (axis < 0 || axis > 3 || n_inputs < 1) return -1;
    int os[4] = {in_shapes4[0], in_shapes4[1], in_shapes4[2], in_shapes4[3]};
    os[axis] = 0;
    for (int i = 0; i < n_inputs; ++i) os[axis] += in_shapes4[i * 4 + axis];
    int off = 0;
    for (int t = 0; t < n_inputs; ++t) {
        const int* s = in_shapes4 + t * 4;
        for (int a = 0; a < s[0]; ++a)
            for (int b = 0; b < s[1]; ++b)
                for (int c = 0; c < s[2]; ++c)
                    for (int d = 0; d < s[3]; ++d) {
                        int o[4] = {a, b, c, d};
                        o[axis] += off;
                        y[((size_t(o[0]) * os[1] + o[1]) * os[2] + o[2]) * os[3] + o[3]] =
                            xs[t][((size_t(a) * s[1] + b) * s[2] + c) * s[3] + d];
                    }
        off += s[axis];
    }
    return 0;
}

int ogle_oracle_transpose(const float* x, const int* is, const int* perm, float* y) {
    int os[4];
    for (int i = 0; i < 4; ++i) os[i] = is[perm[i]];
    for (int a = 0; a < os[0]; ++a)
        for (int b = 0; b < os[1]; ++b)
            for (int c = 0; c < os[2]; ++c)
                for (int d = 0; d < os[3]; ++d) {
                    const int o[4] = {a, b, c, d};
                    int in[4];
                    for (int i = 0; i < 4; ++i) in[perm[i]] = o[i];  // transpose_any4.glsl:44-46
                    y[((size_t(a) * os[1] + b) * os[2] + c) * os[3] + d] =
                        x[((size_t(in[0]) * is[1] + in[1]) * is[2] + in[2]) * is[3] + in[3]];
                }
    return 0;
}

int ogle_oracle_decode(const float* pred, const float* anchors, float* out,
                       int N, int A, const float* var) {
    // ogl_runtime/opengl/core/cpu_functor.cc:129-154; the half-extent products use
    // the double literal 0.5 there, hence the double arithmetic below.
    for (int n = 0; n < N; ++n)
        for (int i = 0; i < A; ++i) {
            const float* p = pred + (size_t(n) * A + i) * 4;
            const float* a = anchors + size_t(i) * 4;
            float* o = out + (size_t(n) * A + i) * 4;
            const float yc = p[1] * var[1] * a[3] + a[1];
            const float xc = p[0] * var[0] * a[2] + a[0];
            const float h = std::exp(p[3] * var[3]) * a[3];
            const float w = std::exp(p[2] * var[2]) * a[2];
            o[0] = float(xc - w * 0.5);
            o[1] = float(yc - h * 0.5);
            o[2] = float(xc + w * 0.5);
            o[3] = float(yc + h * 0.5);
        }
    return 0;
}

namespace {
struct Cand { float score; int cls; int anchor; int rx, ry, rw, rh; };

// ogl_runtime/opengl/examples/ssd/common.cc:57-77 on integer rectangles
float rect_iou(const Cand& a, const Cand& b) {
    const float xmin0 = a.rx, ymin0 = a.ry, xmax0 = a.rx + a.rw, ymax0 = a.ry + a.rh;
    const float xmin1 = b.rx, ymin1 = b.ry, xmax1 = b.rx + b.rw, ymax1 = b.ry + b.rh;
    const float w = std::fmax(0.0f, std::fmin(xmax0, xmax1) - std::fmax(xmin0, xmin1));
    const float h = std::fmax(0.0f, std::fmin(ymax0, ymax1) - std::fmax(ymin0, ymin1));
    const float i = w * h;
    const float u = (xmax0 - xmin0) * (ymax0 - ymin0) + (xmax1 - xmin1) * (ymax1 - ymin1) - i;
    if (u <= 0.0) return 0.0f;
    return i / u;
}
}  // namespace

int ogle_oracle_detect(const float* boxes, const float* logits, int A, int C,
                       int image_w, int image_h, float score_thr, int top_k, float nms_thr,
                       int* out_rect, float* out_score, int* out_class, int* out_anchor) {
    if (C < 2) return -1;
    std::vector<Cand> cands;
    for (int i = 0; i < A; ++i) {
        // detector.cc:176-214
        // `exp` there is the C library's double function (the float argument is promoted,
        // the result rounded back to float): what the reference's file gives when compiled
        // by oracle/ref_detector.cc, against which this function is pinned bit for bit
        const float* s = logits + size_t(i) * C;
        float total = float(std::exp(double(s[0])));
        int max_id = 0;
        float max_prob = 0.f;
        for (int j = 1; j < C; ++j) {
            const float e = float(std::exp(double(s[j])));
            total += e;
            if (max_prob < e) { max_prob = e; max_id = j; }
        }
        const float xmin = boxes[i * 4] * image_w, ymin = boxes[i * 4 + 1] * image_h;
        const float xmax = boxes[i * 4 + 2] * image_w, ymax = boxes[i * 4 + 3] * image_h;
        max_prob /= total;
        if (max_prob > score_thr) {
            Cand c;
            c.score = max_prob; c.cls = max_id; c.anchor = i;
            c.rx = int(xmin); c.ry = int(ymin);              // cv::Rect members are int:
            c.rw = int(xmax - xmin); c.rh = int(ymax - ymin);  // float -> int truncates
            cands.push_back(c);
        }
    }
    // detector.cc:114-125 sorts by score only (unstable); ties are broken here by
    // anchor index so that the order is defined
    std::sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) {
        return a.score > b.score || (a.score == b.score && a.anchor < b.anchor);
    });
    if (top_k < int(cands.size())) cands.resize(top_k);
    // detector.cc:127-148: a box suppresses every later box it overlaps, whether
    // or not it was itself suppressed
    const int n = int(cands.size());
    std::vector<int> label(n, -1);
    for (int i = 0; i < n - 1; ++i)
        for (int j = i + 1; j < n; ++j)
            if (rect_iou(cands[i], cands[j]) > nms_thr) label[j] = 0;
    int kept = 0;
    for (int i = 0; i < n; ++i) {
        if (label[i] != -1) continue;
        out_rect[kept * 4 + 0] = cands[i].rx; out_rect[kept * 4 + 1] = cands[i].ry;
        out_rect[kept * 4 + 2] = cands[i].rw; out_rect[kept * 4 + 3] = cands[i].rh;
        out_score[kept] = cands[i].score;
        out_class[kept] = cands[i].cls;
        out_anchor[kept] = cands[i].anchor;
        ++kept;
    }
    return kept;
}

int ogle_oracle_topk_per_class(const float* logits, int A, int C, float score_thr, int top_k,
                               float* out_score, int* out_anchor, int* out_count) {
    if (C < 2) return -1;
    // softmax as in ogl_runtime/opengl/examples/ssd/common.cc:86-97: exp of the raw
    // logits (no max subtraction), sum in class order, then divide
    std::vector<float> prob(size_t(A) * C);
    for (int i = 0; i < A; ++i) {
        float total = 0.f;
        for (int j = 0; j < C; ++j) { prob[size_t(i) * C + j] = std::exp(logits[size_t(i) * C + j]); total += prob[size_t(i) * C + j]; }
        for (int j = 0; j < C; ++j) prob[size_t(i) * C + j] /= total;
    }
    for (int c = 1; c < C; ++c) {
        std::vector<std::pair<float, int>> v;
        for (int i = 0; i < A; ++i)
            if (prob[size_t(i) * C + c] > score_thr) v.emplace_back(prob[size_t(i) * C + c], i);
        std::sort(v.begin(), v.end(), [](const std::pair<float, int>& a, const std::pair<float, int>& b) {
            return a.first > b.first || (a.first == b.first && a.second < b.second);
        });
        const int n = std::min<int>(top_k, int(v.size()));
        out_count[c - 1] = n;
        for (int i = 0; i < top_k; ++i) {
            out_score[size_t(c - 1) * top_k + i] = i < n ? v[i].first : 0.f;
            out_anchor[size_t(c - 1) * top_k + i] = i < n ? v[i].second : -1;
        }
    }
    return 0;
}


// Detector::Preprocess (examples/ssd/detector.cc:99-109) with OpenCV's 8-bit bilinear
// resize restated (see oracle.h). Horizontal pass in integers scaled by 2^11, vertical
// blend ((b0 * (r0 >> 4)) >> 16) + ((b1 * (r1 >> 4)) >> 16), then (+2) >> 2.
// The two axes treat the border differently: a horizontal tap that falls outside the row
// moves onto the edge pixel with weights (2048, 0); a vertical tap keeps its fractional
// weights and only its row indices are clamped, so both weights then multiply the same
// edge row (the two truncated products can sum to one less than the single product).
// Pinned against cv2.resize in tests/test_oracle.py.
namespace {
void resize_taps(int dst, int src, bool clamp_weights, std::vector<int>* index, std::vector<short>* coef) {
    const double scale = double(src) / dst;
    index->resize(dst);
    coef->resize(size_t(dst) * 2);
    for (int d = 0; d < dst; ++d) {
        float f = float((d + 0.5) * scale - 0.5);
        int s = int(std::floor(f));
        f -= s;
        if (clamp_weights) {
            if (s < 0) { s = 0; f = 0.f; }
            if (s >= src - 1) { s = src - 1; f = 0.f; }
        }
        (*index)[d] = s;
        const float w0 = (1.f - f) * 2048.f, w1 = f * 2048.f;
        (*coef)[d * 2] = short(std::lrintf(w0));       // round half to even, as cvRound does
        (*coef)[d * 2 + 1] = short(std::lrintf(w1));
    }
}
}  // namespace

int ogle_oracle_preprocess_bgr8(const unsigned char* bgr, int src_h, int src_w, int src_row_bytes,
                                float* dst, int dst_h, int dst_w, const float mean_rgb[3]) {
    if (!bgr || !dst || src_h <= 0 || src_w <= 0 || dst_h <= 0 || dst_w <= 0 || src_row_bytes < src_w * 3) return -1;
    std::vector<int> xi, yi;
    std::vector<short> xa, ya;
    resize_taps(dst_w, src_w, true, &xi, &xa);
    resize_taps(dst_h, src_h, false, &yi, &ya);
    for (int y = 0; y < dst_h; ++y) {
        const int y0 = std::min(std::max(yi[y], 0), src_h - 1), y1 = std::min(std::max(yi[y] + 1, 0), src_h - 1);
        const unsigned char* r0 = bgr + size_t(y0) * src_row_bytes;
        const unsigned char* r1 = bgr + size_t(y1) * src_row_bytes;
        const int b0 = ya[y * 2], b1 = ya[y * 2 + 1];
        for (int x = 0; x < dst_w; ++x) {
            const int x0 = xi[x], x1 = std::min(x0 + 1, src_w - 1);
            const int a0 = xa[x * 2], a1 = xa[x * 2 + 1];
            for (int c = 0; c < 3; ++c) {
                const int sc = 2 - c;    // RGB channel c is BGR channel 2 - c
                const int h0 = r0[x0 * 3 + sc] * a0 + r0[x1 * 3 + sc] * a1;
                const int h1 = r1[x0 * 3 + sc] * a0 + r1[x1 * 3 + sc] * a1;
                const int v = (((b0 * (h0 >> 4)) >> 16) + ((b1 * (h1 >> 4)) >> 16) + 2) >> 2;
                const int u8 = v < 0 ? 0 : (v > 255 ? 255 : v);
                dst[(size_t(y) * dst_w + x) * 3 + c] = float(u8) - mean_rgb[c];
            }
        }
    }
    return 0;
}
}  // extern "C"

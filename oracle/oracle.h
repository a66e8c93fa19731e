/* Test infrastructure only. The CPU oracle for the OGLE hot path.
 *
 * Two shared libraries export exactly this interface:
 *   - oracle/liboracle.so       built from oracle/oracle.cc, a CPU restatement of
 *                               the reference's shader and host arithmetic;
 *   - oracle/_ref/libogle_ref.so built from the reference's own source files
 *                               (its GLSL fragment shaders compiled as C++ through
 *                               oracle/glsl_shim.h, and its CPU functors), when the
 *                               reference tree is present at build time.
 * Tests compare the first against the second, and the CUDA path against both.
 * The product library never links, loads or calls either.
 *
 * All buffers are host memory in the reference's PUBLIC layouts: activations
 * NHWC (unpadded), filters OIHW, vectors dense. Padding of the channel dimension
 * to 4 (the reference's NHWC4 / ANY4 / HWN4C4 device layouts) happens inside.
 * Every function returns 0, or a negative value when the request is outside
 * what the reference defines.
 */
#ifndef ORACLE_ORACLE_H_
#define ORACLE_ORACLE_H_
#ifdef __cplusplus
extern "C" {
#endif

/* Number of host threads the library will use (OpenMP). */
int ogle_oracle_threads(void);
void ogle_oracle_set_threads(int n);

/* act: 0 none, 1 clip(min,max), 2 relu.  Variant selection (general / pointwise /
 * depthwise / grouped) follows Conv2DKernel::SelectKernel,
 * ogl_runtime/opengl/nn/kernels/conv2d.cc:19-51. bias may be NULL. */
int ogle_oracle_conv2d(const float* x, const float* w_oihw, const float* bias, float* y,
                       int N, int H, int W, int C, int K, int kernel, int stride, int pad,
                       int dilation, int group, int act, float min_value, float max_value);

/* type: 0 max, 1 average (divides by kernel*kernel, padding included);
 * ogl_runtime/opengl/nn/glsl/pool.glsl:19-66. */
int ogle_oracle_pool(const float* x, float* y, int N, int H, int W, int C,
                     int kernel, int stride, int pad, int type);

/* ogl_runtime/opengl/nn/glsl/batchnorm.glsl:18-32 */
int ogle_oracle_batchnorm(const float* x, const float* gamma, const float* beta,
                          const float* mean, const float* var, float* y,
                          int N, int H, int W, int C, float eps);

/* relu.glsl, clip.glsl, binary.glsl: elementwise over n floats */
int ogle_oracle_relu(const float* x, float* y, long n);
int ogle_oracle_clip(const float* x, float* y, long n, float lo, float hi);
int ogle_oracle_add(const float* a, const float* b, float* y, long n);

/* Y[M,N] = alpha*A[M,K]*(transB ? B[N,K]^T : B[K,N]) + beta*C.
 * bias_mode: 0 none, 1 C is [M,N], 2 C is [N] broadcast over rows.
 * ogl_runtime/opengl/nn/glsl/gemm.glsl:24-95. */
int ogle_oracle_gemm(const float* A, const float* B, const float* C, float* Y,
                     int M, int K, int N, int transB, float alpha, float beta, int bias_mode);

/* Concatenate n_inputs 4-D tensors (shapes left-padded with 1s, 4 ints each)
 * along axis (0..3). ogl_runtime/opengl/nn/kernels/concat.cc:53-96. */
int ogle_oracle_concat(int n_inputs, const float* const* xs, const int* in_shapes4,
                       int axis, float* y);

/* y[o0,o1,o2,o3] with out dim i = in dim perm[i].
 * ogl_runtime/opengl/nn/glsl/transpose_any4.glsl:13-69 */
int ogle_oracle_transpose(const float* x, const int* in_shape4, const int* perm4, float* y);

/* SSD centre-size decode to corner boxes; pred [N,A,4], anchors [A,4] (cx,cy,w,h)
 * shared by all images, out [N,A,4] (xmin,ymin,xmax,ymax).
 * ogl_runtime/opengl/core/cpu_functor.cc:129-154 */
int ogle_oracle_decode(const float* pred, const float* anchors, float* out,
                       int N, int A, const float* variances4);

/* Layout conversions, ogl_runtime/opengl/core/cpu_functor.cc:10-127.
 * pad4:  [rows,last] -> [rows, round_up(last,4)] zero-filled
 * unpad4: inverse
 * prepack_filter: OIHW -> [(kh*kw)*ceil(O/4)][ceil(I/4)*4][4]  (HWN4C4)
 * unpack_filter: inverse */
int ogle_oracle_pad4(const float* x, float* y, long rows, int last);
int ogle_oracle_unpad4(const float* x, float* y, long rows, int last);
int ogle_oracle_prepack_filter(const float* w_oihw, float* packed, int O, int I, int kh, int kw);
int ogle_oracle_unpack_filter(const float* packed, float* w_oihw, int O, int I, int kh, int kw);

/* Detector post-process of the SSD example, one image:
 * softmax over C classes, best class among 1..C-1, keep score > thr, sort by
 * score descending (ties: lower anchor index first), keep top_k, greedy NMS on
 * boxes truncated to integer pixel rectangles.
 * ogl_runtime/opengl/examples/ssd/detector.cc:114-228, common.cc:57-77.
 * boxes [A,4] normalised corners, logits [A,C]. Outputs hold up to top_k rows:
 * out_rect (x,y,w,h ints), out_score, out_class, out_anchor. Returns the number
 * of detections kept, or a negative value. Only liboracle.so implements this;
 * _ref/libogle_ref.so exports the reference's own compiled post-process as
 * ogle_ref_detect (oracle/ref_detector.cc), against which this one is pinned. */
int ogle_oracle_detect(const float* boxes, const float* logits, int A, int C,
                       int image_w, int image_h, float score_thr, int top_k, float nms_thr,
                       int* out_rect, float* out_score, int* out_class, int* out_anchor);

/* Standard SSD per-class selection (an extension over the reference's
 * best-class rule): softmax, then for every foreground class c in 1..C-1 keep
 * anchors with p[c] > thr, ordered by (score desc, anchor asc), at most top_k.
 * out_score/out_anchor are [C-1, top_k]; out_count[C-1]. Only liboracle.so
 * implements this. */
int ogle_oracle_topk_per_class(const float* logits, int A, int C, float score_thr, int top_k,
                               float* out_score, int* out_anchor, int* out_count);

/* Detector::Preprocess, ogl_runtime/opengl/examples/ssd/detector.cc:99-109:
 * BGR -> RGB, resize of the 8-bit image to dst_h x dst_w, conversion to float,
 * minus mean (R, G, B). The resize is OpenCV's (a third-party dependency that is
 * not in the reference tree; the reference pins no version): cv::resize with the
 * default INTER_LINEAR on 8-bit data, restated here from its published
 * behaviour - pixel-centre alignment ((d + 0.5) * scale - 0.5), weights rounded to
 * 11 fractional bits, rows blended in 32-bit fixed point with rounding to nearest;
 * horizontal taps outside the row become the edge pixel, vertical ones keep their
 * weights on the clamped row. PINNED: bit-exact against cv2.cvtColor + cv2.resize
 * (OpenCV 4.13) outputs committed under tests/golden/ and against the installed
 * OpenCV where there is one (tests/test_oracle.py).
 * Output: dst_h x dst_w x 3 floats (NHWC, unpadded). Only liboracle.so implements this. */
int ogle_oracle_preprocess_bgr8(const unsigned char* bgr, int src_h, int src_w, int src_row_bytes,
                                float* dst, int dst_h, int dst_w, const float mean_rgb[3]);

#ifdef __cplusplus
}
#endif
#endif /* ORACLE_ORACLE_H_ */

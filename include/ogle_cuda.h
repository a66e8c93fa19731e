/* ogle_cuda.h - C ABI of the B200 (sm_100a) backend for the OGLE graph runtime's
 * data-parallel hot path: conv2d family with fused bias/BN/activation, gemm,
 * pooling, elementwise, concat, layout conversion and the SSD box decoder and
 * post-process.
 *
 * The reference runtime (kl456123/OGLE) has no foreign-function interface: each
 * operator's Kernel::Compute binds OpenGL textures and draws. Every entry point
 * below is what such a Compute (or a Context copy function) calls instead, and
 * its comment cites the reference code it replaces, by path inside that project.
 *
 * Conventions
 *  - All pointers are DEVICE pointers unless a name ends in _host.
 *  - Activations use ONE layout: [N][H][W][Cs] fp32 with Cs = channel stride in
 *    floats, Cs >= round_up(C,4) and Cs % 4 == 0. This is the byte layout of the
 *    reference's NHWC4 textures and of its ANY4 textures for 4-D shapes
 *    (ogl_runtime/opengl/core/tensor_format.cc:308-337). Lanes C..Cs-1 of a
 *    tensor produced here are zero unless a wider stride was requested for an
 *    in-place concat.
 *  - Every function enqueues work on `stream` and returns immediately. None
 *    allocates device memory, synchronises or aborts. Return value: OGLE_OK or
 *    a negative OgleStatus.
 *  - One host thread per device; calls for different streams/devices may run
 *    concurrently from different threads.
 */
#ifndef OGLE_CUDA_H_
#define OGLE_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ogle_stream_t; /* == cudaStream_t */

typedef enum {
    OGLE_OK = 0,
    OGLE_ERR_INVALID = -1,     /* bad argument (shape, stride, null pointer) */
    OGLE_ERR_UNSUPPORTED = -2, /* outside what the reference defines          */
    OGLE_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed            */
    OGLE_ERR_ALIGNMENT = -4,   /* pointer or stride not 16-byte aligned        */
    OGLE_ERR_DEVICE = -5,      /* not an sm_100 device / no device             */
    OGLE_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up           */
} OgleStatus;

/* Arithmetic used by the dense contractions (conv2d general/pointwise, gemm). */
typedef enum {
    OGLE_MATH_FP32 = 0,   /* CUDA-core fp32 FMA                                         */
    OGLE_MATH_TF32 = 1,   /* tcgen05 kind::tf32, one pass (10-bit mantissa operands)    */
    OGLE_MATH_TF32X3 = 2  /* hi/lo operand split, three products (one TF32 pass + one BF16
                             pass of the two cross terms): fp32-grade results           */
} OgleMathMode;

typedef enum { OGLE_ACT_NONE = 0, OGLE_ACT_CLIP = 1, OGLE_ACT_RELU = 2 } OgleActivation;

const char* ogle_cuda_status_string(int status);
/* Library version and the GPU architecture it was built for ("sm_100a"). */
const char* ogle_cuda_build_info(void);
/* Number of kernels this library has launched in this process (all streams). */
uint64_t ogle_cuda_launch_count(void);
/* Last CUDA error string seen by this library on the calling thread. */
const char* ogle_cuda_last_error(void);
/* Device-side status word of the tensor-core kernels: 0, or the code of the first
 * bounded wait that gave up (the launch then produced no valid output). Reading
 * synchronises the device; clear resets it. */
int ogle_cuda_device_status(void);
int ogle_cuda_clear_device_status(void);
/* The raw status word: which wait gave up (1 producer, 2 MMA issuer, 3 operand split,
 * 4 epilogue, 5 accumulator hand-back); 0 when none did. Synchronises the device. */
int ogle_cuda_device_status_detail(void);
/* Programmatic dependent launches for the kernels launched after this call (process-wide): each kernel's
 * prologue (barrier set-up, tensor-memory allocation, descriptor prefetch) may then run while its predecessor
 * on the stream drains; every kernel waits for its predecessor's results before its first global access. Pays
 * when the launches are short (5 % at one image per step, 1-4 % up to 16), costs 1-2 % when they are long: the
 * runtime turns it on for sessions whose tensors hold less than 1 GB. The environment variable OGLE_PDL (0/1), when set, overrides it.
 * Captured CUDA graphs keep what was in force when they were captured. */
int ogle_cuda_set_overlapped_launches(int on);

/* How many times a role of the tensor-core kernels polls for its turn before it gives up, for
 * the launches that follow on any stream (process-wide). polls < 0 restores the default (2^22,
 * tens of milliseconds); 0 makes every such wait give up at once. It exists to exercise the
 * give-up path without a fault: a launch whose waits run out writes no valid output, sets the
 * status word, waits for its own copies and multiplies in flight (those waits keep the full
 * bound), frees its tensor memory and returns, and the device stays usable. No counterpart in
 * the reference, whose only failure handling is glGetError -> abort (utils/macros.cc:21-28). */
int ogle_cuda_set_wait_limit(long polls);

/* ------------------------------------------------------------------ conv2d */
/* Mirrors the uniform set of Conv2DKernel::Compute,
 * ogl_runtime/opengl/nn/kernels/conv2d.cc:116-167, plus the output placement
 * fields that let a producer write straight into a concat consumer. */
typedef struct {
    int N;
    int in_hwc[3];   /* H, W, C of the input   */
    int out_hwc[3];  /* Ho, Wo, K of the output */
    int kernel, stride, pad, dilation, group;
    int has_bias;
    int act;         /* OgleActivation */
    float min_value, max_value;
    int in_channel_stride;   /* floats per input pixel; 0 = round_up(C,4)   */
    int out_channel_stride;  /* floats per output pixel; 0 = round_up(K,4)  */
    int out_channel_offset;  /* first output channel lands here (mult of 4) */
    int math_mode;           /* OgleMathMode */
    int n_tile;              /* tensor-core path: output channels per tile (a multiple of 32, at most
                                256 and round_up(K,32)); 0 = chosen by the library. Results do not
                                depend on it bit for bit (each output value sums its reduction in the
                                same order); a caller may time the candidates and keep the fastest. */
    int split;               /* tensor-core path: ranges the reduction is split into (1 = not split, up to
                                16; more than 2, or any with an activation, needs the scratch of
                                ogle_cuda_conv2d_ws); 0 = chosen by the library. Unlike n_tile this changes the
                                order in which a value's partial sums are added. */
    int channels_on_m;       /* tensor-core path, at most 128 output channels, unsplit reduction: 2 = keep the
                                accumulator transposed (filters on the 128-row side of the multiply, 256 pixels per
                                instruction), which halves the tensor-core instructions of layers with 64-128 output
                                channels; 1 = no, 0 = chosen by the library. Ignored where it cannot run. */
    int sm_pair;             /* tensor-core path: 2 = compute tiles of 256 pixels on pairs of SMs (each SM of a
                                pair loads half of the filter tile; needs n_tile a multiple of 64 and an unsplit
                                reduction, else ignored), 1 = one SM per tile, 0 = chosen by the library.
                                Results do not depend on it bit for bit. */
} OgleConvParams;

/* Output size rule of Conv2DKernel::InferOutputShape (conv2d.cc:169-195).
 * Fills p->out_hwc from the other fields. */
int ogle_cuda_conv2d_infer(OgleConvParams* p);

/* Bytes of the device-side packed filter for these parameters. */
size_t ogle_cuda_conv2d_filter_bytes(const OgleConvParams* p);

/* Re-lays an OIHW filter [K][C/group][k][k] (device) into the layout the conv
 * kernels read. Replaces the NCHW->HWN4C4 upload pass,
 * ogl_runtime/opengl/core/context.cc:123-154 with nchw_to_hwn4c4.glsl. Run once
 * per model, like the reference's "ready" pre-compute (fbo_session.cc:240-245). */
int ogle_cuda_conv2d_prepack(const OgleConvParams* p, const float* w_oihw, void* packed,
                             ogle_stream_t stream);

/* y = act(conv(x, w) + bias). Variant choice follows Conv2DKernel::SelectKernel
 * (conv2d.cc:19-51): pointwise, depthwise, grouped, general. Replaces
 * conv2d.glsl, conv2d_pw.glsl, conv2d_dw.glsl, conv2d_grp.glsl and their _any4
 * twins. bias: K floats (may be NULL when has_bias == 0). */
int ogle_cuda_conv2d(const OgleConvParams* p, const float* x, const void* packed_filter,
                     const float* bias, float* y, ogle_stream_t stream);

/* y = act(conv(x, w) + bias + residual): the convolution, the Add of a residual block and the activation that
 * follows it in one pass (replaces the binary.glsl pass of nn/kernels/binary.cc and, with act != none, the relu.glsl /
 * clip.glsl pass after it; same fp32 operations in the same order as the separate passes, so the result is bit-identical
 * to them). residual: a tensor with the output's pixels, residual_stride floats per pixel (0 = round_up(K,4)), channel c of
 * the convolution at residual[pixel * residual_stride + c]. Served by the tensor-core path only
 * (ogle_cuda_conv2d_residual_supported: math_mode TF32 or TF32X3, >= 16 input channels); OGLE_ERR_UNSUPPORTED otherwise -
 * the caller then runs ogle_cuda_conv2d and ogle_cuda_add_act. */
int ogle_cuda_conv2d_residual_supported(const OgleConvParams* p);
int ogle_cuda_conv2d_residual(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                              const float* residual, int residual_stride, float* y, ogle_stream_t stream);

/* The same with scratch memory lent by the caller (device memory, 16-byte aligned, at least
 * ogle_cuda_conv2d_workspace_bytes(p), which is 0 for most layers). Layers with a long reduction
 * and few output tiles - 3x3 heads on small feature maps, the whole network at batch 1 - then split
 * their reduction over up to 16 blocks per tile: each block stores its partial tile into its own
 * slice of the scratch and a second small kernel adds the slices in a fixed order, then bias and
 * activation (bit-reproducible; any activation). Without scratch such layers split in two at
 * most, and only without an activation. The scratch may be reused as soon as the stream has
 * passed this call. */
size_t ogle_cuda_conv2d_workspace_bytes(const OgleConvParams* p);
int ogle_cuda_conv2d_ws(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                        float* y, void* workspace, size_t workspace_bytes, ogle_stream_t stream);

/* Name of the device kernel that ogle_cuda_conv2d launches for these parameters
 * (for profiles and reports; "" when the parameters are invalid). */
const char* ogle_cuda_conv2d_kernel_name(const OgleConvParams* p);

/* Two convolutions that read the same input with the same window (kernel, stride,
 * pad, dilation, activation, group 1) as ONE pass over the input: the SSD box and
 * class heads, which the reference draws as two Conv2DKernel::Compute passes
 * (conv2d.cc:116-167) over the same feature map. The caller stacks the two OIHW
 * filters into one of out_hwc[2] = second_offset + K2 rows, where
 * second_offset = K1 rounded up to a multiple of 32 and the rows in between are
 * zero, packs it with ogle_cuda_conv2d_prepack under the same params, and stacks
 * the biases the same way. y_first receives channels [0, K1) as a tensor of K1
 * channels (padded to 4), y_second channels [second_offset, out_hwc[2]) as a tensor
 * of K2 channels. The arithmetic per output value is that of ogle_cuda_conv2d,
 * up to the order in which partial sums are added (the two forms may split a
 * long reduction into different numbers of ranges). Tensor-core modes only: ogle_cuda_conv2d_pair_supported says
 * whether these params are served (else run the two convolutions separately). */
int ogle_cuda_conv2d_pair_supported(const OgleConvParams* p);
int ogle_cuda_conv2d_pair(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                          int first_channels, int second_offset, float* y_first, float* y_second,
                          ogle_stream_t stream);
/* ogle_cuda_conv2d_pair with scratch memory, as ogle_cuda_conv2d_ws. */
size_t ogle_cuda_conv2d_pair_workspace_bytes(const OgleConvParams* p, int first_channels, int second_offset);
int ogle_cuda_conv2d_pair_ws(const OgleConvParams* p, const float* x, const void* packed_filter, const float* bias,
                             int first_channels, int second_offset, float* y_first, float* y_second, void* workspace,
                             size_t workspace_bytes, ogle_stream_t stream);

/* -------------------------------------------------------------------- pool */
/* PoolKernel::Compute, ogl_runtime/opengl/nn/kernels/pool.cc:55-79 + pool.glsl.
 * type: 0 max (all-padding window gives 0), 1 average (divides by kernel^2,
 * padding included), 2 global average (kernel := H, requires H == W). */
typedef struct {
    int N;
    int in_hwc[3];
    int out_hwc[3];
    int kernel, stride, pad, type;
    int in_channel_stride, out_channel_stride; /* 0 = round_up(C,4) */
} OglePoolParams;
int ogle_cuda_pool_infer(OglePoolParams* p);
int ogle_cuda_pool(const OglePoolParams* p, const float* x, float* y, ogle_stream_t stream);

/* ------------------------------------------------------------- elementwise */
/* BatchNormKernel::Compute, nn/kernels/batchnorm.cc:30-78 + batchnorm.glsl:
 * (x-mean)/sqrt(var+eps)*gamma+beta, params are C floats each. */
int ogle_cuda_batchnorm(const float* x, const float* gamma, const float* beta, const float* mean,
                        const float* var, float* y, long pixels, int C, int channel_stride,
                        float eps, ogle_stream_t stream);
/* relu.glsl / clip.glsl / binary.glsl over n floats (n % 4 == 0). */
int ogle_cuda_relu(const float* x, float* y, long n, ogle_stream_t stream);
int ogle_cuda_clip(const float* x, float* y, long n, float lo, float hi, ogle_stream_t stream);
int ogle_cuda_add(const float* a, const float* b, float* y, long n, ogle_stream_t stream);
/* binary.glsl followed by relu.glsl or clip.glsl (a residual block's Add -> Relu) in one pass:
 * y = act(a + b), act an OgleActivation; bit-identical to the two passes. */
int ogle_cuda_add_act(const float* a, const float* b, float* y, long n, int act, float lo, float hi,
                      ogle_stream_t stream);

/* -------------------------------------------------------------------- gemm */
/* GemmKernel::Compute, nn/kernels/gemm.cc:25-65 + gemm.glsl:
 * Y[M,N] = alpha*A[M,K]*(transB ? B[N,K]^T : B[K,N]) + beta*C.
 * Row strides (lda, ldb, ldc, ldy, in floats) are round_up(cols,4) for the
 * reference's ANY4 layout. bias_mode: 0 none, 1 C is [M,N] (ldc), 2 C is [N]
 * broadcast over rows (the reference defines this only for M == 1). */
typedef struct {
    int M, K, N;
    int transB;
    float alpha, beta;
    int bias_mode;
    int lda, ldb, ldc, ldy;
    int math_mode; /* OgleMathMode */
} OgleGemmParams;
int ogle_cuda_gemm(const OgleGemmParams* p, const float* A, const float* B, const float* C,
                   float* Y, ogle_stream_t stream);

/* B operand re-laid for the tensor-core path: K-major [round_up(N,128)][round_up(K,32)]
 * split into hi (10 mantissa bits) and lo (remainder) halves. Like the conv filter
 * packing, it is done once for a constant B (the usual case: Gemm weights are model
 * constants) and replaces the ANY -> ANY4 upload pass of context.cc:135-141. */
size_t ogle_cuda_gemm_packed_b_bytes(const OgleGemmParams* p);
int ogle_cuda_gemm_pack_b(const OgleGemmParams* p, const float* B, void* packed, ogle_stream_t stream);
/* ogle_cuda_gemm with B given in packed form (math_mode TF32 or TF32X3; FP32 is
 * served from the raw B by ogle_cuda_gemm). */
int ogle_cuda_gemm_packed(const OgleGemmParams* p, const float* A, const void* packed_b, const float* C,
                          float* Y, ogle_stream_t stream);

/* ogle_cuda_gemm for a B that is NOT a constant (both operands produced at run
 * time): the tensor-core modes need B re-laid and split, so the caller lends
 * `workspace` (device memory, >= ogle_cuda_gemm_packed_b_bytes(p), 16-byte aligned).
 * The call packs B into it and multiplies, both on `stream`; the workspace may be
 * reused as soon as the stream has passed this call. */
int ogle_cuda_gemm_ws(const OgleGemmParams* p, const float* A, const float* B, const float* C, float* Y,
                      void* workspace, size_t workspace_bytes, ogle_stream_t stream);

/* ogle_cuda_gemm_ws with the packing scratch in a fixed device array inside the
 * library instead of a caller's workspace. It has no counterpart in the reference.
 * It allocates nothing, on any call: the scratch is a file-scope device array of
 * OGLE_GEMM_STATIC_MAX_BYTES. A problem whose packed B
 * (ogle_cuda_gemm_packed_b_bytes) is larger returns OGLE_ERR_UNSUPPORTED with the
 * sizes in ogle_cuda_last_error(); use ogle_cuda_gemm_ws then.
 * The first call on each device resolves the array's address (set-up; make it with
 * that device current and before any stream capture); later calls only launch.
 * All calls on a device share the one array: calls that may execute concurrently
 * (two streams without an event between them) race on it. Nothing in the array has
 * to be cleared between calls. */
#define OGLE_GEMM_STATIC_MAX_BYTES (8u << 20)
size_t ogle_cuda_gemm_static_max_bytes(void);
int ogle_cuda_gemm_static(const OgleGemmParams* p, const float* A, const float* B, const float* C, float* Y,
                          ogle_stream_t stream);

/* ------------------------------------------------------------------ concat */
/* ConcatKernel::Compute, nn/kernels/concat.cc:53-96 + concat_multi.glsl.
 * Shapes are 4-D (left-padded with 1s, as AmendShape does); last dimension of
 * every tensor is stored padded to a multiple of 4. One pass, each input read
 * once and written once. A NULL entry of the input array means that slice is already in
 * place (its producer wrote it there): it is neither read nor written. */
#define OGLE_MAX_CONCAT_INPUTS 16
typedef struct {
    int n_inputs;
    int axis;                                   /* 0..3 */
    int in_shapes[OGLE_MAX_CONCAT_INPUTS][4];
} OgleConcatParams;
int ogle_cuda_concat(const OgleConcatParams* p, const float* const* inputs_host_array,
                     float* y, ogle_stream_t stream);

/* -------------------------------------------------- layout / glue kernels */
/* ANY -> ANY4 / NHWC -> NHWC4 upload conversion and back
 * (Context::CopyCPUTensorToDevice / CopyDeviceTensorToCPU,
 * ogl_runtime/opengl/core/context.cc:123-185; any_to_any4.glsl, any4_to_any.glsl):
 * [rows][last] dense <-> [rows][stride] with zero fill. stride 0 = round_up(last,4). */
int ogle_cuda_pad4(const float* dense, float* padded, long rows, int last, int stride,
                   ogle_stream_t stream);
int ogle_cuda_unpad4(const float* padded, float* dense, long rows, int last, int stride,
                     ogle_stream_t stream);
/* Detector::Preprocess (examples/ssd/detector.cc:99-109) for one image: 8-bit BGR
 * (device memory, rows src_row_bytes apart) -> RGB, bilinear resize to
 * dst_h x dst_w with OpenCV's 8-bit INTER_LINEAR arithmetic (the cv::resize call
 * the reference makes), to float, minus mean_rgb; written as [dst_h][dst_w][4]
 * floats (the NHWC4 slot of one image of the network input; lane 3 = 0). */
int ogle_cuda_preprocess_bgr8(const unsigned char* bgr, int src_h, int src_w, int src_row_bytes,
                              float* dst_nhwc4, int dst_h, int dst_w, const float mean_rgb[3],
                              ogle_stream_t stream);
/* The same for n_images images in ONE launch. The images sit in one device byte buffer;
 * descs_device (device memory, n_images entries) says where each starts and how large it
 * is. Image i is written to dst_nhwc4 + i * dst_h * dst_w * 4. The sizes are not checked
 * on the device: the caller filled the table. */
typedef struct OgleImageDesc {
    long long offset;      /* byte offset of the image's first pixel in the buffer */
    int height, width;     /* pixels */
    int row_bytes;         /* distance between rows, >= 3 * width */
    int reserved;
} OgleImageDesc;
int ogle_cuda_preprocess_bgr8_batch(const unsigned char* bgr_base, const OgleImageDesc* descs_device, int n_images,
                                    float* dst_nhwc4, int dst_h, int dst_w, const float mean_rgb[3],
                                    ogle_stream_t stream);
/* NCHW dense -> NHWC4 (for callers holding NCHW images). */
int ogle_cuda_nchw_to_nhwc4(const float* nchw, float* nhwc4, int N, int C, int H, int W,
                            ogle_stream_t stream);
/* TransposeKernel (nn/kernels/transpose.cc:73-90 + transpose_any4.glsl): 4-D
 * permute, out dim i = in dim perm[i]; both sides padded on their last dim. */
int ogle_cuda_transpose(const float* x, float* y, const int in_shape[4], const int perm[4],
                        ogle_stream_t stream);
/* ReshapeKernel / FlattenKernel (nn/kernels/reshape.cc:30-46 + reshape_any4.glsl):
 * same logical element order, different padded last dimension. */
int ogle_cuda_reshape(const float* x, float* y, long n_elements, int in_last, int out_last,
                      ogle_stream_t stream);
/* The same copy with its output rows laid out for a consumer that concatenates: output row r
 * is written at y + (r / rows_per_block) * block_stride + (r % rows_per_block) * round_up(out_last,4)
 * (floats; block_stride % 4 == 0). With rows_per_block = the rows one image contributes and
 * block_stride = the floats of one image in the concatenated tensor, the copy lands in its
 * slice of that tensor and the concat pass for it (concat.cc:73-96) is not needed. */
int ogle_cuda_reshape_placed(const float* x, float* y, long n_elements, int in_last, int out_last,
                             long rows_per_block, long block_stride, ogle_stream_t stream);

/* --------------------------------------------------------------------- SSD */
/* functor::SSDBBoxDecoder (ogl_runtime/opengl/core/functor.cc:96-143 +
 * decoder.glsl): pred [N][A][4] deltas, anchors [A][4] (cx,cy,w,h) shared by all
 * images, out [N][A][4] corners (xmin,ymin,xmax,ymax). */
int ogle_cuda_ssd_decode(const float* pred, const float* anchors, float* out, int N, int A,
                         const float variances[4], ogle_stream_t stream);

/* Detector post-process (ogl_runtime/opengl/examples/ssd/detector.cc:114-228):
 * the reference does this on the CPU after reading back boxes and logits.
 * mode 0 (reference rule): softmax, best foreground class per anchor, keep
 *   score > score_thr, top_k by score over the image (ties: lower anchor
 *   first), then the reference's greedy NMS on integer pixel rectangles when
 *   nms_thr > 0. Output rows per image: top_k.
 * mode 1 (per-class, standard SSD): softmax, per foreground class keep
 *   score > score_thr and the top_k by score. Output rows per image:
 *   (C-1)*top_k. No NMS.
 * logits [N][A][logit_stride] (logit_stride >= C); boxes [N][A][4] corners.
 * Outputs (device): out_score [N][rows] (0 where empty), out_anchor [N][rows]
 * (-1 where empty), out_class [N][rows], out_box [N][rows][4] (mode 0: integer
 * pixel rect x,y,w,h as floats; mode 1: the corner box), out_count [N] (mode 0)
 * or [N][C-1] (mode 1). */
typedef struct {
    int N, A, C;
    int logit_stride;
    int mode;
    float score_thr;
    int top_k;       /* <= 256 */
    float nms_thr;   /* mode 0 only; <= 0 disables NMS */
    int image_w, image_h; /* mode 0: scale to pixels */
    /* mode 0, optional (NULL = every image is image_w x image_h): device table of n
     * entries whose width/height give the pixel size of image n's ORIGINAL frame. The
     * reference scales boxes by the raw frame it was handed, not by the network input
     * (origin_input_sizes_, detector.cc:102,179-180), so frames of different sizes in one
     * batch need their own scale. Only width and height of an entry are read. */
    const OgleImageDesc* frame_sizes;
} OgleDetectParams;
int ogle_cuda_ssd_detect(const OgleDetectParams* p, const float* logits, const float* boxes,
                         float* out_score, int* out_anchor, int* out_class, float* out_box,
                         int* out_count, ogle_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* OGLE_CUDA_H_ */

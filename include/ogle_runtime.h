/* ogle_runtime.h - C ABI of the host runtime (libogle_rt.so): the graph session
 * and the SSD detector, for callers that do not link the C++ classes.
 *
 * The reference runtime is a C++ library with no foreign-function interface;
 * each entry point below names the C++ member it wraps, which in turn mirrors a
 * member of the reference (cited by path inside kl456123/OGLE).
 *
 * Error behaviour: the reference aborts the process on any failed check. Here
 * the same conditions come back as a negative return value and
 * ogle_rt_last_error() holds the message for the calling thread.
 */
#ifndef OGLE_RUNTIME_H_
#define OGLE_RUNTIME_H_
#include <stddef.h>
#include <stdint.h>
#include "ogle_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OgleSession OgleSession;
typedef struct OgleDetector OgleDetector;

/* dlxnet.TensorProto.DataFormat values (ogl_runtime/opengl/core/dlxnet.proto:8-29) */
enum { OGLE_FMT_NCHW = 0, OGLE_FMT_NHWC = 1, OGLE_FMT_NHWC4 = 3, OGLE_FMT_HWN4C4 = 4, OGLE_FMT_ANY = 5, OGLE_FMT_ANY4 = 6 };

const char* ogle_rt_last_error(void);
/* Operator names in the kernel registry, '\n'-separated
 * (REGISTER_KERNEL_WITH_NAME, ogl_runtime/opengl/core/kernel_registry.h:36-42). */
const char* ogle_rt_registered_kernels(void);

/* FBOSession(), ogl_runtime/opengl/core/fbo_session.h:13-15. device < 0 keeps the
 * current CUDA device; stream NULL creates a private stream. */
OgleSession* ogle_session_create(int device, ogle_stream_t stream);
void ogle_session_destroy(OgleSession* s);
/* "math_mode" (OgleMathMode), "use_graph" (0/1), "fuse_siblings" (0/1: sibling convolutions
 * of one input as one pass), "fuse_activations" (0/1: a Relu/Clip that is the only reader of an
 * Add runs in the Add's pass; the Add's own tensor is then not readable), "fuse_concats" (0/1: a Conv
 * or re-padding Reshape whose result only a Concat reads writes into its slice of the Concat's tensor; a
 * Concat with every slice written that way is dropped; the producers' own tensors are then not readable),
 * "fuse_residuals" (0/1: an Add one of whose operands is a convolution's result that nothing else reads runs in
 * that convolution's pass, with the Relu the Add may have taken over; the convolution's and the Add's own tensors
 * are then not readable),
 * "tune" (0/1: after set-up every convolution served by the tensor cores times its tile widths on its own
 * tensors and keeps the fastest; the reduction of a layer may then be split differently from session to
 * session, i.e. results can differ in the last bits between sessions, never between runs of one),
 * "streams" (1..8: streams the captured graph's independent
 * branches are recorded on; 1 = file order, as the reference runs). Set before the first run. */
int ogle_session_set_option(OgleSession* s, const char* key, int value);
/* FBOSession::LoadGraph(path) / LoadGraph(ModelProto), fbo_session.cc:62-124. */
int ogle_session_load_graph_file(OgleSession* s, const char* path);
int ogle_session_load_graph_bytes(OgleSession* s, const void* data, size_t size);
/* FBOSession::Run(NamedTensorList), fbo_session.cc:127-156. Each input is a dense
 * host tensor (data, shape, rank, dformat). Asynchronous; host buffers must stay
 * valid until ogle_session_synchronize or a get_output call. */
int ogle_session_run(OgleSession* s, int n_inputs, const char* const* names, const float* const* data_host,
                     const int* const* shapes, const int* ranks, const int* dformats);
/* Same, with inputs already on the device in the padded NHWC4/ANY4 layout. */
int ogle_session_run_device(OgleSession* s, int n_inputs, const char* const* names, const float* const* data_device);
int ogle_session_synchronize(OgleSession* s);
/* FBOSession::FindTensorByName: shape (up to 8 dims), rank, device data format, device pointer. */
int ogle_session_tensor_info(OgleSession* s, const char* name, int* shape8, int* rank, int* dformat, void** device_ptr);
/* FBOSession::GetOutputs for one tensor, fbo_session.cc:276-301. dformat is "NHWC",
 * "NCHW", "ANY", "NHWC4", "ANY4" or "HWN4C4". Synchronises. */
int ogle_session_get_output(OgleSession* s, const char* name, const char* dformat, float* out_host, size_t capacity_floats);
int ogle_session_num_active_kernels(OgleSession* s);
/* Concat inputs that their producers write in place (option "fuse_concats"). */
int ogle_session_num_placed(OgleSession* s);
/* Residual Adds that run in a convolution's pass (option "fuse_residuals"). */
int ogle_session_num_residuals(OgleSession* s);
/* Branches of the captured graph that run beside the stream of their predecessors
 * (option "streams" > 1); 0 before the capture or for a chain. */
int ogle_session_num_branches(OgleSession* s);
int ogle_session_graph_captured(OgleSession* s);
size_t ogle_session_device_bytes(OgleSession* s);
/* One eager pass with per-node timing; writes "name\ttype\tkernel\tms\n" rows into buf. */
int ogle_session_profile(OgleSession* s, int n_inputs, const char* const* names, const float* const* data_host,
                         const int* const* shapes, const int* ranks, const int* dformats, char* buf, size_t buf_size);

/* Detector::Create / Detect, ogl_runtime/opengl/examples/ssd/detector.cc:24-47,275-295.
 * mode 0: reference rule; mode 1: per-class top-k. Tensor names default to
 * "input", "cls_logits", "box_preds", "anchors" when NULL. */
OgleDetector* ogle_detector_create(int device, ogle_stream_t stream, const char* model_path, int mode, float score_thr,
                                   int top_k, float nms_thr, int math_mode, const char* input_name,
                                   const char* logits_name, const char* boxes_name, const char* anchors_name);
void ogle_detector_destroy(OgleDetector* d);
/* Enqueue upload + network + decode + post-process + copy-back for N preprocessed NHWC images. */
int ogle_detector_detect_async(OgleDetector* d, const float* images_nhwc_host, int N, int H, int W);
/* Raw frames instead of preprocessed floats: N 8-bit BGR images (host memory, tightly
 * packed rows, any sizes). Upload as bytes, then on the device channel swap, 8-bit bilinear
 * resize to H x W, float, minus mean_rgb[3] (Detector::Preprocess, detector.cc:99-109),
 * then as ogle_detector_detect_async. Retired by ogle_detector_wait. */
int ogle_detector_detect_bgr8_async(OgleDetector* d, const unsigned char* const* images, const int* heights,
                                    const int* widths, int N, int H, int W, const float* mean_rgb);
/* Same for images already on the device as [N][H][W][4] floats (channel 3 zero).
 * The session must have been sized by one ogle_detector_detect_async call of the
 * same shape. copy_back 0 leaves the detections on the device. */
int ogle_detector_detect_device_async(OgleDetector* d, const float* images_nhwc4_device, int N, int H, int W, int copy_back);
/* Wait for it and copy the results out. rows = top_k (mode 0) or (C-1)*top_k (mode 1).
 * Any output pointer may be NULL. count holds N (mode 0) or N*(C-1) ints. */
int ogle_detector_wait(OgleDetector* d, float* score, int* anchor, int* cls, float* box, int* count);
int ogle_detector_info(OgleDetector* d, int* num_anchors, int* num_classes, int* rows, size_t* h2d_bytes, size_t* d2h_bytes);
OgleSession* ogle_detector_session(OgleDetector* d);
/* Result memory of the caller's for the detector's two pipeline slots (pinned or
 * CUDA-registered host memory, 16-byte aligned, bytes_each >= the total of
 * ogle_detector_result_layout for the batch): detections are copied from the device
 * straight into it, and ogle_detector_wait still blocks until they are there. With the
 * slots inside a region from ogle_host_shared_open, the process that owns a batch sharded
 * over several per-GPU processes reads every shard's detections in place, where the
 * reference's single process reads its one read-back (detector.cc:242-273). Call before
 * the first detect call. */
int ogle_detector_use_result_buffers(OgleDetector* d, void* slot0_host, void* slot1_host, size_t bytes_each);
/* Byte offsets of score [N][rows] f32, anchor [N][rows] i32, class [N][rows] i32,
 * box [N][rows][4] f32, count [N][counts_per_image] i32 inside one result block, and its
 * total size: offsets6 = {score, anchor, class, box, count, total}. */
int ogle_detector_result_layout(int mode, int num_classes, int top_k, int N, size_t* offsets6, int* rows,
                                int* counts_per_image);

/* The session's stream planner on its own (pure host logic; option "streams"): nodes in
 * execution order, each with the memory spans [lo, hi) it reads and writes, given as n_spans
 * records (span_node[i], span_lo[i], span_hi[i], span_is_write[i]). Writes lane[n_nodes] (the
 * stream of each node) and, when waits is not NULL, waits[i * n_nodes + j] = 1 where node i
 * must wait for node j recorded on another stream. Returns the number of branches, -1 on bad
 * arguments. */
int ogle_rt_plan_streams(int n_nodes, int n_spans, const int* span_node, const unsigned long long* span_lo,
                         const unsigned long long* span_hi, const int* span_is_write, int streams, int* lane,
                         unsigned char* waits);

/* Host placement for one process (or thread) per GPU. No counterpart in the reference, which
 * runs one GL context on one thread (ogl_runtime/opengl/core/init.cc:21-43).
 * ogle_host_bind_to_device: narrows the calling thread's CPU affinity to the CPUs of the
 * NUMA node the device's PCIe function belongs to (among those it may already use) and makes
 * its later page allocations, pinned buffers included, prefer that node. Call it before
 * allocating the buffers that feed the device. Always returns 0; *numa_node is -1 and the
 * other outputs 0 where the topology is unknown or nothing could be changed. */
int ogle_host_bind_to_device(int device, int* numa_node, int* cpus_bound, int* memory_preferred);
/* Pinned host memory for the buffers a caller uploads from: anonymous memory advised to use
 * 2 MB pages (transparent huge pages where the host grants them), zeroed, registered with
 * CUDA. Uploads from it cost fewer IOMMU translations than from 4 KB pages, which shows when
 * several GPUs upload at once. NULL on failure. Call on the thread whose device context is
 * current; free only with ogle_host_free_pinned. */
void* ogle_host_alloc_pinned(size_t bytes);
void ogle_host_free_pinned(void* p);
/* Bytes of the mapping holding p that the kernel backs with 2 MB pages right now (0 = none
 * were granted, or unknown). */
size_t ogle_host_huge_page_bytes(const void* p);
/* A named region of host memory shared by the per-GPU processes of one box (POSIX shared
 * memory; name starts with '/'). create != 0 makes and zero-fills it, otherwise an existing
 * one is mapped; pin != 0 registers the mapping with CUDA in the calling process (device
 * context current), so that uploads from it and result copies into it are asynchronous.
 * One batch is then written once by its owner, uploaded slice by slice by every process, and
 * the detections land where the owner reads them: the host-side scatter and gather of an
 * image-sharded batch without a copy between processes. NULL on failure
 * (ogle_rt_last_error). ogle_host_shared_close unmaps; unlink != 0 also removes the name. */
void* ogle_host_shared_open(const char* name, size_t bytes, int create, int pin);
void ogle_host_shared_close(void* p, int unlink);
/* One asynchronous host-to-device copy on `stream` (the upload half of
 * Context::CopyCPUTensorToDevice, core/context.cc:123-154, without the layout pass): what the
 * detector issues per batch, exposed so that the bare upload rate of a host buffer can be
 * measured beside the full pipeline. */
int ogle_host_upload_async(void* dst_device, const void* src_host, size_t bytes, ogle_stream_t stream);
/* Parses a sysfs CPU list ("0-3,8,10-11"); writes up to `capacity` entries, returns the count. */
int ogle_host_parse_cpulist(const char* text, int* cpus, int capacity);

#ifdef __cplusplus
}
#endif
#endif /* OGLE_RUNTIME_H_ */

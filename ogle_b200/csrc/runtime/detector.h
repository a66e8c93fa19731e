// Detector: the SSD example's pipeline (ogl_runtime/opengl/examples/ssd/detector.h)
// without OpenCV: session->Run on preprocessed NHWC float images, box decode, and
// the post-process (softmax, threshold, top-k, NMS) - which the reference runs on
// the CPU after reading back all boxes and logits - as one device kernel, so that
// only the detections cross back to the host.
#ifndef OGLE_RUNTIME_DETECTOR_H_
#define OGLE_RUNTIME_DETECTOR_H_
#include "fbo_session.h"
#include "functor.h"

namespace ogle {

struct DetectorOptions {
    std::string model_name;
    int topk = 100;                 // detector.cc:34-37
    float nms_threshold = 0.45f;
    float score_threshold = 0.3f;
    std::vector<float> variances = {0.1f, 0.1f, 0.2f, 0.2f};
    // mode 0: the reference's rule (best foreground class, image-wide top-k, NMS);
    // mode 1: per-class top-k (standard SSD), no NMS
    int mode = 0;
    TensorNameList input_names = {"input"};
    TensorNameList output_names = {"cls_logits", "box_preds", "anchors"};
};

// Views into the detector's pinned result buffer (no copy): valid until the same pipeline
// slot is reused, i.e. until kDepth further calls have been issued.
struct DetectionBatch {
    int images = 0;
    int rows = 0;                       // rows per image
    int counts_per_image = 0;           // 1 (mode 0) or C-1 (mode 1)
    const float* score = nullptr;       // [N][rows]
    const int* anchor = nullptr;        // [N][rows]
    const int* cls = nullptr;           // [N][rows]
    const float* box = nullptr;         // [N][rows][4]
    const int* count = nullptr;         // [N][counts_per_image]
};

class Detector {
public:
    Detector(const DetectorOptions& options, Context* context);
    ~Detector();
    // images: host NHWC [N,H,W,3] floats, already mean-subtracted (Preprocess of
    // detector.cc:99-109 needs an image library and is the caller's). Enqueues the
    // upload, the network, decode, post-process and the copy of the detections into
    // pinned memory, and returns. Up to kDepth calls may be in flight: the upload of
    // call i+1 (copy stream) overlaps the network of call i (compute stream), and the
    // copy-back of call i overlaps the network of call i+1. Pinned host memory makes
    // the copies truly asynchronous. The host buffer must stay valid until the Wait()
    // that retires this call.
    void DetectAsync(const float* images_nhwc, int N, int H, int W);
    // Raw frames: N 8-bit BGR images of any sizes in host memory (pinned memory makes the
    // copies asynchronous). Each is uploaded as bytes and turned into the H x W network
    // input on the device - channel swap, 8-bit bilinear resize, float, minus mean_rgb -
    // which is Detector::Preprocess + Detect of the reference (detector.cc:99-109, 275-295).
    // Pipelined and retired by Wait() like DetectAsync.
    void DetectBGR8Async(const unsigned char* const* images, const int* heights, const int* widths, int N, int H, int W,
                         const float mean_rgb[3]);
    // Same, for images that already sit on the device in the padded NHWC4 layout
    // [N][H][W][4]. copy_back = false leaves the detections on the device and enqueues
    // nothing for Wait(); with copy_back the call is retired by Wait() like DetectAsync.
    // Not pipelined: call it only with no DetectAsync in flight.
    void DetectDeviceAsync(const float* images_nhwc4_device, int N, int H, int W, bool copy_back);
    // Retires the OLDEST call in flight: blocks until its detections are on the host.
    const DetectionBatch& Wait();
    // Result memory of the caller's: the detections of the two pipeline slots are copied to
    // slot0 / slot1 (pinned or CUDA-registered host memory of at least ResultBytes(N) each)
    // instead of buffers the detector allocates - e.g. this process's part of a region that
    // several per-GPU processes share, so that the process collecting a sharded batch reads
    // every shard's detections in place. Call before the first Detect*; the memory must
    // outlive the detector.
    void UseResultBuffers(void* slot0, void* slot1, size_t bytes_each);
    // Byte layout of one call's result block for N images: offsets of score, anchor, class,
    // box and count, and the total (what Wait() hands out as DetectionBatch views).
    struct ResultLayout { size_t score, anchor, cls, box, count, total; int rows, counts_per_image; };
    static ResultLayout LayoutFor(int mode, int num_classes, int topk, int N);
    int in_flight() const { return int(pending_.size()); }
    static constexpr int kDepth = 2;

    FBOSession* session() { return session_.get(); }
    int num_classes() const { return num_classes_; }
    int num_anchors() const { return num_anchors_; }
    int rows() const { return rows_; }
    size_t h2d_bytes() const { return h2d_bytes_; }
    size_t d2h_bytes() const { return d2h_bytes_; }

private:
    struct Slot {
        float* stage = nullptr;      // dense NHWC upload target on the device
        unsigned char* bytes = nullptr;   // raw 8-bit frames of one call (DetectBGR8Async)
        size_t bytes_capacity = 0;
        void* desc_host = nullptr;   // pinned table of the frames' places and sizes in `bytes`
        size_t desc_capacity = 0;    // entries
        void* out_dev = nullptr;     // score | anchor | cls | box | count, contiguous
        void* out_host = nullptr;    // pinned mirror
        bool out_host_external = false;   // the caller's memory (UseResultBuffers): not freed here
        void* ev_h2d = nullptr;      // upload landed (copy-in stream)
        void* ev_pad = nullptr;      // staging buffer consumed (compute stream)
        void* ev_done = nullptr;     // post-process finished (compute stream)
        void* ev_d2h = nullptr;      // detections on the host (copy-out stream)
    };
    void EnsureSession(int N, int H, int W, const float* images_nhwc);
    void Allocate(int N, int H, int W);
    void Release();
    void PostProcess(Slot& slot, int N, int H, int W, const OgleImageDesc* frames_device);
    DetectorOptions options_;
    Context* context_;
    std::unique_ptr<FBOSession> session_;
    int num_classes_ = 0, num_anchors_ = 0, batch_ = 0, rows_ = 0, counts_per_image_ = 0;
    float* boxes_ = nullptr;          // decoded [N][A][4]
    Slot slots_[kDepth];
    int next_slot_ = 0;
    std::vector<int> pending_;
    void* copy_in_ = nullptr;         // cudaStream_t
    void* copy_out_ = nullptr;
    size_t out_bytes_ = 0, off_anchor_ = 0, off_cls_ = 0, off_box_ = 0, off_count_ = 0;
    size_t h2d_bytes_ = 0, d2h_bytes_ = 0, stage_bytes_ = 0;
    DetectionBatch result_;
    void* external_result_[kDepth] = {nullptr, nullptr};
    size_t external_result_bytes_ = 0;
};

}  // namespace ogle
#endif

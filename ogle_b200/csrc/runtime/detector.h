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

struct DetectionBatch {
    int rows = 0;                       // rows per image
    std::vector<float> score;           // [N][rows]
    std::vector<int> anchor, cls;       // [N][rows]
    std::vector<float> box;             // [N][rows][4]
    std::vector<int> count;             // [N] (mode 0) or [N][C-1] (mode 1)
};

class Detector {
public:
    Detector(const DetectorOptions& options, Context* context);
    ~Detector();
    // images: host NHWC [N,H,W,3] floats, already mean-subtracted (Preprocess of
    // detector.cc:99-109 needs an image library and is the caller's). Enqueues the
    // upload, the network, decode and post-process, and the copies of the results
    // into pinned staging; Wait() then exposes them.
    void DetectAsync(const float* images_nhwc, int N, int H, int W);
    // Same, for images that already sit on the device in the padded NHWC4 layout
    // [N][H][W][4]; copy_back = false leaves the detections on the device.
    void DetectDeviceAsync(const float* images_nhwc4_device, int N, int H, int W, bool copy_back);
    // Blocks until the last DetectAsync finished; results are valid until the next call.
    const DetectionBatch& Wait();
    FBOSession* session() { return session_.get(); }
    int num_classes() const { return num_classes_; }
    int num_anchors() const { return num_anchors_; }
    int rows() const { return rows_; }
    size_t h2d_bytes() const { return h2d_bytes_; }
    size_t d2h_bytes() const { return d2h_bytes_; }
    // device pointers of the last post-process outputs (valid after the first call)
    const float* device_boxes() const { return boxes_; }

private:
    void AllocateOutputs(int N);
    void PostProcess(int N, int H, int W, bool copy_back);
    DetectorOptions options_;
    Context* context_;
    std::unique_ptr<FBOSession> session_;
    int num_classes_ = 0, num_anchors_ = 0, batch_ = 0, rows_ = 0, counts_per_image_ = 0;
    float* boxes_ = nullptr;          // decoded [N][A][4]
    void* out_dev_ = nullptr;         // score | anchor | cls | box | count, contiguous
    void* out_host_ = nullptr;        // pinned mirror
    size_t out_bytes_ = 0, off_anchor_ = 0, off_cls_ = 0, off_box_ = 0, off_count_ = 0;
    size_t h2d_bytes_ = 0, d2h_bytes_ = 0;
    DetectionBatch result_;
};

}  // namespace ogle
#endif

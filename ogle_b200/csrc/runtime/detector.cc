#include "detector.h"

#include <cuda_runtime.h>
#include <cstring>

namespace ogle {

#define OGLE_RT_CUDA(call)                                                              \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) OGLE_FATAL() << #call << ": " << cudaGetErrorString(e_); \
    } while (0)

static cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
static cudaEvent_t E(void* e) { return reinterpret_cast<cudaEvent_t>(e); }

Detector::Detector(const DetectorOptions& options, Context* context) : options_(options), context_(context) {
    OGLE_CHECK_EQ(options_.output_names.size(), 3u);
    OGLE_CHECK_EQ(options_.input_names.size(), 1u);
    context_->MakeCurrent();
    session_.reset(new FBOSession(context_));
    session_->LoadGraph(options_.model_name);
    cudaStream_t a, b;
    OGLE_RT_CUDA(cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking));
    OGLE_RT_CUDA(cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking));
    copy_in_ = a;
    copy_out_ = b;
    for (Slot& s : slots_) {
        cudaEvent_t e[4];
        for (auto& x : e) OGLE_RT_CUDA(cudaEventCreateWithFlags(&x, cudaEventDisableTiming));
        s.ev_h2d = e[0]; s.ev_pad = e[1]; s.ev_done = e[2]; s.ev_d2h = e[3];
    }
}

void Detector::Release() {
    if (boxes_) cudaFree(boxes_);
    boxes_ = nullptr;
    for (Slot& s : slots_) {
        if (s.stage) cudaFree(s.stage);
        if (s.bytes) cudaFree(s.bytes);
        s.bytes = nullptr; s.bytes_capacity = 0;
        if (s.desc_host) cudaFreeHost(s.desc_host);
        s.desc_host = nullptr; s.desc_capacity = 0;
        if (s.out_dev) cudaFree(s.out_dev);
        if (s.out_host && !s.out_host_external) cudaFreeHost(s.out_host);
        s.stage = nullptr; s.out_dev = nullptr; s.out_host = nullptr; s.out_host_external = false;
    }
}

Detector::~Detector() {
    context_->MakeCurrent();
    cudaDeviceSynchronize();
    Release();
    for (Slot& s : slots_) {
        cudaEventDestroy(E(s.ev_h2d)); cudaEventDestroy(E(s.ev_pad));
        cudaEventDestroy(E(s.ev_done)); cudaEventDestroy(E(s.ev_d2h));
    }
    cudaStreamDestroy(S(copy_in_));
    cudaStreamDestroy(S(copy_out_));
}

void Detector::Allocate(int N, int H, int W) {
    const size_t stage_bytes = size_t(N) * H * W * 3 * sizeof(float);
    if (N == batch_ && stage_bytes == stage_bytes_) return;
    OGLE_CHECK(pending_.empty()) << "the batch shape may only change with no call in flight";
    OGLE_RT_CUDA(cudaDeviceSynchronize());
    Release();
    const ResultLayout L = LayoutFor(options_.mode, num_classes_, options_.topk, N);
    rows_ = L.rows;
    counts_per_image_ = L.counts_per_image;
    off_anchor_ = L.anchor; off_cls_ = L.cls; off_box_ = L.box; off_count_ = L.count;
    out_bytes_ = L.total;
    OGLE_RT_CUDA(cudaMalloc(&boxes_, size_t(N) * num_anchors_ * 16));
    for (int i = 0; i < kDepth; ++i) {
        Slot& s = slots_[i];
        OGLE_RT_CUDA(cudaMalloc(&s.stage, stage_bytes));
        OGLE_RT_CUDA(cudaMalloc(&s.out_dev, out_bytes_));
        if (external_result_[i]) {
            OGLE_CHECK_GE(external_result_bytes_, out_bytes_) << "result buffers given to UseResultBuffers are too small";
            s.out_host = external_result_[i];
            s.out_host_external = true;
        } else {
            OGLE_RT_CUDA(cudaMallocHost(&s.out_host, out_bytes_));
        }
    }
    batch_ = N;
    stage_bytes_ = stage_bytes;
}

Detector::ResultLayout Detector::LayoutFor(int mode, int num_classes, int topk, int N) {
    ResultLayout L;
    L.rows = mode == 0 ? topk : (num_classes - 1) * topk;
    L.counts_per_image = mode == 0 ? 1 : num_classes - 1;
    const size_t n = size_t(N) * size_t(L.rows);
    L.score = 0;
    L.anchor = n * 4;
    L.cls = L.anchor + n * 4;
    L.box = (L.cls + n * 4 + 15) / 16 * 16;
    L.count = L.box + n * 16;
    L.total = L.count + size_t(N) * size_t(L.counts_per_image) * 4;
    return L;
}

void Detector::UseResultBuffers(void* slot0, void* slot1, size_t bytes_each) {
    OGLE_CHECK(batch_ == 0 && pending_.empty()) << "UseResultBuffers must come before the first Detect call";
    OGLE_CHECK(slot0 && slot1 && slot0 != slot1 && bytes_each > 0);
    OGLE_CHECK((reinterpret_cast<uintptr_t>(slot0) & 15) == 0 && (reinterpret_cast<uintptr_t>(slot1) & 15) == 0)
        << "result buffers must be 16-byte aligned";
    external_result_[0] = slot0;
    external_result_[1] = slot1;
    external_result_bytes_ = bytes_each;
}

void Detector::EnsureSession(int N, int H, int W, const float* images_nhwc) {
    if (batch_ == 0 || !session_->FindTensorByName(options_.input_names[0])) {
        // first call: let the session see an input once so that it sizes every tensor
        // (FBOSession::Setup, fbo_session.cc:168-252); detector.cc:235-240
        std::vector<float> zeros;
        if (!images_nhwc) {
            zeros.assign(size_t(N) * H * W * 3, 0.f);
            images_nhwc = zeros.data();
        }
        Tensor input(Tensor::DT_FLOAT, IntList{N, H, W, 3}, const_cast<float*>(images_nhwc), dlxnet::TensorProto::NHWC);
        session_->Setup({{options_.input_names[0], &input}});
        context_->Synchronize();
        Tensor* cls_logits = session_->FindTensorByName(options_.output_names[0]);
        Tensor* box_preds = session_->FindTensorByName(options_.output_names[1]);
        OGLE_CHECK(cls_logits && box_preds);
        OGLE_CHECK_EQ(cls_logits->shape().size(), 3u);   // detector.cc:152-155
        OGLE_CHECK_EQ(box_preds->shape().size(), 3u);
        num_anchors_ = box_preds->shape()[1];
        num_classes_ = cls_logits->shape()[2];
        OGLE_CHECK_EQ(cls_logits->shape()[1], num_anchors_);
    }
    Tensor* in = session_->FindTensorByName(options_.input_names[0]);
    OGLE_CHECK(in->shape() == (IntList{N, H, W, 3})) << "input shape differs from the one the session was sized for";
    Allocate(N, H, W);
}

void Detector::DetectBGR8Async(const unsigned char* const* images, const int* heights, const int* widths, int N, int H,
                               int W, const float mean_rgb[3]) {
    context_->MakeCurrent();
    OGLE_CHECK(images && heights && widths && mean_rgb && N > 0);
    OGLE_CHECK_LT(int(pending_.size()), kDepth) << "retire a call with Wait() before issuing another";
    cudaStream_t compute = S(context_->stream());
    EnsureSession(N, H, W, nullptr);
    Tensor* in = session_->FindTensorByName(options_.input_names[0]);
    Slot& slot = slots_[next_slot_];
    // device byte buffer of the call: [table of OgleImageDesc, one per image][the images, back to back]
    const size_t table_bytes = (size_t(N) * sizeof(OgleImageDesc) + 255) / 256 * 256;
    if (size_t(N) > slot.desc_capacity) {
        // the slot is not pending (checked above), so nothing still reads its old table
        if (slot.desc_host) cudaFreeHost(slot.desc_host);
        OGLE_RT_CUDA(cudaMallocHost(&slot.desc_host, table_bytes));
        slot.desc_capacity = table_bytes / sizeof(OgleImageDesc);
    }
    OgleImageDesc* table = static_cast<OgleImageDesc*>(slot.desc_host);
    size_t total = table_bytes;
    for (int i = 0; i < N; ++i) {
        OGLE_CHECK(images[i] && heights[i] > 0 && widths[i] > 0) << "image " << i;
        table[i].offset = static_cast<long long>(total);
        table[i].height = heights[i]; table[i].width = widths[i];
        table[i].row_bytes = widths[i] * 3; table[i].reserved = 0;
        total += size_t(heights[i]) * widths[i] * 3;
    }
    // this slot's byte buffer was last read two calls ago (ev_pad); growing it needs that done
    if (total > slot.bytes_capacity) {
        OGLE_RT_CUDA(cudaEventSynchronize(E(slot.ev_pad)));
        if (slot.bytes) cudaFree(slot.bytes);
        OGLE_RT_CUDA(cudaMalloc(&slot.bytes, total));
        slot.bytes_capacity = total;
    }
    OGLE_RT_CUDA(cudaStreamWaitEvent(S(copy_in_), E(slot.ev_pad), 0));
    OGLE_RT_CUDA(cudaMemcpyAsync(slot.bytes, table, size_t(N) * sizeof(OgleImageDesc), cudaMemcpyHostToDevice, S(copy_in_)));
    // images that follow one another in host memory (frames of one buffer) go up as one copy
    for (int i = 0; i < N;) {
        size_t run = size_t(heights[i]) * widths[i] * 3;
        int j = i + 1;
        while (j < N && images[j] == images[j - 1] + size_t(heights[j - 1]) * widths[j - 1] * 3) {
            run += size_t(heights[j]) * widths[j] * 3;
            ++j;
        }
        OGLE_RT_CUDA(cudaMemcpyAsync(slot.bytes + table[i].offset, images[i], run, cudaMemcpyHostToDevice, S(copy_in_)));
        i = j;
    }
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_h2d), S(copy_in_)));
    h2d_bytes_ = total - table_bytes + size_t(N) * sizeof(OgleImageDesc);
    OGLE_RT_CUDA(cudaStreamWaitEvent(compute, E(slot.ev_h2d), 0));
    OGLE_CUDA_OK(ogle_cuda_preprocess_bgr8_batch(slot.bytes, reinterpret_cast<const OgleImageDesc*>(slot.bytes), N,
                                                 in->device<float>(), H, W, mean_rgb, context_->stream()));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_pad), compute));
    session_->RunDevice({});
    // the reference scales each frame's boxes by that frame's own size (detector.cc:102,179-180);
    // the table at the head of the byte buffer holds them
    PostProcess(slot, N, H, W, reinterpret_cast<const OgleImageDesc*>(slot.bytes));
    OGLE_RT_CUDA(cudaStreamWaitEvent(S(copy_out_), E(slot.ev_done), 0));
    OGLE_RT_CUDA(cudaMemcpyAsync(slot.out_host, slot.out_dev, out_bytes_, cudaMemcpyDeviceToHost, S(copy_out_)));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_d2h), S(copy_out_)));
    d2h_bytes_ = out_bytes_;
    pending_.push_back(next_slot_);
    next_slot_ = (next_slot_ + 1) % kDepth;
}

void Detector::DetectAsync(const float* images_nhwc, int N, int H, int W) {
    context_->MakeCurrent();
    OGLE_CHECK_LT(int(pending_.size()), kDepth) << "retire a call with Wait() before issuing another";
    cudaStream_t compute = S(context_->stream());
    EnsureSession(N, H, W, images_nhwc);
    Tensor* in = session_->FindTensorByName(options_.input_names[0]);
    Slot& slot = slots_[next_slot_];
    // upload on the copy stream, once the compute stream has consumed this slot's last upload
    OGLE_RT_CUDA(cudaStreamWaitEvent(S(copy_in_), E(slot.ev_pad), 0));
    OGLE_RT_CUDA(cudaMemcpyAsync(slot.stage, images_nhwc, stage_bytes_, cudaMemcpyHostToDevice, S(copy_in_)));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_h2d), S(copy_in_)));
    h2d_bytes_ = stage_bytes_;
    // pad to NHWC4 into the session's input tensor (Context::CopyCPUTensorToDevice's second half)
    OGLE_RT_CUDA(cudaStreamWaitEvent(compute, E(slot.ev_h2d), 0));
    OGLE_CUDA_OK(ogle_cuda_pad4(slot.stage, in->device<float>(), long(N) * H * W, 3, 0, context_->stream()));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_pad), compute));
    session_->RunDevice({});
    PostProcess(slot, N, H, W, nullptr);      // preprocessed input: the frame is the network input
    // copy the detections back on their own stream
    OGLE_RT_CUDA(cudaStreamWaitEvent(S(copy_out_), E(slot.ev_done), 0));
    OGLE_RT_CUDA(cudaMemcpyAsync(slot.out_host, slot.out_dev, out_bytes_, cudaMemcpyDeviceToHost, S(copy_out_)));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_d2h), S(copy_out_)));
    d2h_bytes_ = out_bytes_;
    pending_.push_back(next_slot_);
    next_slot_ = (next_slot_ + 1) % kDepth;
}

void Detector::DetectDeviceAsync(const float* images_nhwc4_device, int N, int H, int W, bool copy_back) {
    context_->MakeCurrent();
    OGLE_CHECK(pending_.empty()) << "DetectDeviceAsync is not pipelined: retire the calls in flight first";
    Tensor* in = session_->FindTensorByName(options_.input_names[0]);
    OGLE_CHECK(in != nullptr && batch_ == N) << "run DetectAsync once before DetectDeviceAsync (it sizes the session)";
    OGLE_CHECK(in->shape() == (IntList{N, H, W, 3})) << "device input does not match the session's input shape";
    session_->RunDevice({{options_.input_names[0], images_nhwc4_device}});
    h2d_bytes_ = 0;
    Slot& slot = slots_[next_slot_];
    PostProcess(slot, N, H, W, nullptr);
    d2h_bytes_ = 0;
    if (!copy_back) return;    // stream-ordered on the compute stream; nothing for Wait() to retire
    OGLE_RT_CUDA(cudaMemcpyAsync(slot.out_host, slot.out_dev, out_bytes_, cudaMemcpyDeviceToHost, S(context_->stream())));
    d2h_bytes_ = out_bytes_;
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_d2h), S(context_->stream())));
    pending_.push_back(next_slot_);
    next_slot_ = (next_slot_ + 1) % kDepth;
}

void Detector::PostProcess(Slot& slot, int N, int H, int W, const OgleImageDesc* frames_device) {
    cudaStream_t compute = S(context_->stream());
    Tensor* cls_logits = session_->FindTensorByName(options_.output_names[0]);
    Tensor* box_preds = session_->FindTensorByName(options_.output_names[1]);
    Tensor* anchors = session_->FindTensorByName(options_.output_names[2]);
    OGLE_CHECK(cls_logits && box_preds && anchors);
    OGLE_CHECK_EQ(cls_logits->shape()[0], N);
    // detector.cc:242-258: GPU box decode into a cached tensor
    Tensor decoded(IntList{N, num_anchors_, 4}, dlxnet::TensorProto::ANY4, boxes_);
    Tensor anchors2d(IntList{num_anchors_, 4}, dlxnet::TensorProto::ANY4, anchors->device<float>());
    OGLE_CHECK_EQ(anchors->num_elements(), size_t(num_anchors_) * 4);
    functor::SSDBBoxDecoder()(context_, box_preds, &anchors2d, &decoded, options_.variances);
    // detector.cc:150-228 on the device
    OgleDetectParams p;
    std::memset(&p, 0, sizeof(p));
    p.N = N; p.A = num_anchors_; p.C = num_classes_;
    p.logit_stride = UpRound4(num_classes_);
    p.mode = options_.mode;
    p.score_thr = options_.score_threshold;
    p.top_k = options_.topk;
    p.nms_thr = options_.nms_threshold;
    p.image_w = W; p.image_h = H;
    p.frame_sizes = options_.mode == 0 ? frames_device : nullptr;
    // this slot's output buffer must have been copied out by its previous user
    OGLE_RT_CUDA(cudaStreamWaitEvent(compute, E(slot.ev_d2h), 0));
    char* d = static_cast<char*>(slot.out_dev);
    OGLE_CUDA_OK(ogle_cuda_ssd_detect(&p, cls_logits->device<float>(), boxes_, reinterpret_cast<float*>(d),
                                      reinterpret_cast<int*>(d + off_anchor_), reinterpret_cast<int*>(d + off_cls_),
                                      reinterpret_cast<float*>(d + off_box_), reinterpret_cast<int*>(d + off_count_),
                                      context_->stream()));
    OGLE_RT_CUDA(cudaEventRecord(E(slot.ev_done), compute));
}

const DetectionBatch& Detector::Wait() {
    context_->MakeCurrent();
    OGLE_CHECK(!pending_.empty()) << "Wait() without a call in flight";
    const int idx = pending_.front();
    pending_.erase(pending_.begin());
    Slot& slot = slots_[idx];
    OGLE_RT_CUDA(cudaEventSynchronize(E(slot.ev_d2h)));
    const char* h = static_cast<const char*>(slot.out_host);
    result_.images = batch_;
    result_.rows = rows_;
    result_.counts_per_image = counts_per_image_;
    result_.score = reinterpret_cast<const float*>(h);
    result_.anchor = reinterpret_cast<const int*>(h + off_anchor_);
    result_.cls = reinterpret_cast<const int*>(h + off_cls_);
    result_.box = reinterpret_cast<const float*>(h + off_box_);
    result_.count = reinterpret_cast<const int*>(h + off_count_);
    return result_;
}

}  // namespace ogle

#include "detector.h"

#include <cuda_runtime.h>
#include <cstring>

namespace ogle {

#define OGLE_RT_CUDA(call)                                                              \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) OGLE_FATAL() << #call << ": " << cudaGetErrorString(e_); \
    } while (0)

Detector::Detector(const DetectorOptions& options, Context* context) : options_(options), context_(context) {
    OGLE_CHECK_EQ(options_.output_names.size(), 3u);
    OGLE_CHECK_EQ(options_.input_names.size(), 1u);
    session_.reset(new FBOSession(context_));
    session_->LoadGraph(options_.model_name);
}

Detector::~Detector() {
    context_->MakeCurrent();
    if (boxes_) cudaFree(boxes_);
    if (out_dev_) cudaFree(out_dev_);
    if (out_host_) cudaFreeHost(out_host_);
}

void Detector::AllocateOutputs(int N) {
    if (N == batch_) return;
    context_->Synchronize();
    if (boxes_) cudaFree(boxes_);
    if (out_dev_) cudaFree(out_dev_);
    if (out_host_) cudaFreeHost(out_host_);
    boxes_ = nullptr; out_dev_ = nullptr; out_host_ = nullptr;
    rows_ = options_.mode == 0 ? options_.topk : (num_classes_ - 1) * options_.topk;
    counts_per_image_ = options_.mode == 0 ? 1 : num_classes_ - 1;
    const size_t n = size_t(N) * rows_;
    off_anchor_ = n * 4;
    off_cls_ = off_anchor_ + n * 4;
    off_box_ = (off_cls_ + n * 4 + 15) / 16 * 16;
    off_count_ = off_box_ + n * 16;
    out_bytes_ = off_count_ + size_t(N) * counts_per_image_ * 4;
    OGLE_RT_CUDA(cudaMalloc(&boxes_, size_t(N) * num_anchors_ * 16));
    OGLE_RT_CUDA(cudaMalloc(&out_dev_, out_bytes_));
    OGLE_RT_CUDA(cudaMallocHost(&out_host_, out_bytes_));
    batch_ = N;
}

void Detector::DetectAsync(const float* images_nhwc, int N, int H, int W) {
    context_->MakeCurrent();
    Tensor input(Tensor::DT_FLOAT, IntList{N, H, W, 3}, const_cast<float*>(images_nhwc), dlxnet::TensorProto::NHWC);
    session_->Run({{options_.input_names[0], &input}});          // detector.cc:235-240
    h2d_bytes_ = input.num_elements() * sizeof(float);
    PostProcess(N, H, W, true);
}

void Detector::DetectDeviceAsync(const float* images_nhwc4_device, int N, int H, int W, bool copy_back) {
    context_->MakeCurrent();
    Tensor* in = session_->FindTensorByName(options_.input_names[0]);
    OGLE_CHECK(in != nullptr) << "run DetectAsync once before DetectDeviceAsync (it sizes the session)";
    OGLE_CHECK(in->shape() == (IntList{N, H, W, 3})) << "device input does not match the session's input shape";
    session_->RunDevice({{options_.input_names[0], images_nhwc4_device}});
    h2d_bytes_ = 0;
    PostProcess(N, H, W, copy_back);
}

void Detector::PostProcess(int N, int H, int W, bool copy_back) {
    Tensor* cls_logits = session_->FindTensorByName(options_.output_names[0]);
    Tensor* box_preds = session_->FindTensorByName(options_.output_names[1]);
    Tensor* anchors = session_->FindTensorByName(options_.output_names[2]);
    OGLE_CHECK(cls_logits && box_preds && anchors);
    OGLE_CHECK_EQ(cls_logits->shape().size(), 3u);   // detector.cc:152-155
    OGLE_CHECK_EQ(box_preds->shape().size(), 3u);
    num_anchors_ = box_preds->shape()[1];
    num_classes_ = cls_logits->shape()[2];
    OGLE_CHECK_EQ(cls_logits->shape()[1], num_anchors_);
    OGLE_CHECK_EQ(cls_logits->shape()[0], N);
    AllocateOutputs(N);
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
    char* d = static_cast<char*>(out_dev_);
    OGLE_CUDA_OK(ogle_cuda_ssd_detect(&p, cls_logits->device<float>(), boxes_, reinterpret_cast<float*>(d),
                                      reinterpret_cast<int*>(d + off_anchor_), reinterpret_cast<int*>(d + off_cls_),
                                      reinterpret_cast<float*>(d + off_box_), reinterpret_cast<int*>(d + off_count_),
                                      context_->stream()));
    d2h_bytes_ = 0;
    if (copy_back) {
        OGLE_RT_CUDA(cudaMemcpyAsync(out_host_, out_dev_, out_bytes_, cudaMemcpyDeviceToHost,
                                     reinterpret_cast<cudaStream_t>(context_->stream())));
        d2h_bytes_ = out_bytes_;
    }
}

const DetectionBatch& Detector::Wait() {
    context_->MakeCurrent();
    context_->Synchronize();
    const size_t n = size_t(batch_) * rows_;
    const char* h = static_cast<const char*>(out_host_);
    result_.rows = rows_;
    result_.score.assign(reinterpret_cast<const float*>(h), reinterpret_cast<const float*>(h) + n);
    result_.anchor.assign(reinterpret_cast<const int*>(h + off_anchor_), reinterpret_cast<const int*>(h + off_anchor_) + n);
    result_.cls.assign(reinterpret_cast<const int*>(h + off_cls_), reinterpret_cast<const int*>(h + off_cls_) + n);
    result_.box.assign(reinterpret_cast<const float*>(h + off_box_), reinterpret_cast<const float*>(h + off_box_) + n * 4);
    result_.count.assign(reinterpret_cast<const int*>(h + off_count_),
                         reinterpret_cast<const int*>(h + off_count_) + size_t(batch_) * counts_per_image_);
    return result_;
}

}  // namespace ogle

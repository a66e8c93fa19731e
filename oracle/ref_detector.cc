// Test infrastructure only (never linked into or loaded by the product libraries).
//
// The reference's own detection post-process compiled for the CPU: its
// ogl_runtime/opengl/examples/ssd/detector.cc (Detector::GenerateBoxInfo :150-228,
// GetTopK :114-125, NMS :127-148) and common.cc (iou :57-77, softmax :86-97) are
// #included below unmodified, read in place from the reference tree, against the stand-in
// headers under oracle/ref_shim/ (OpenCV types, a session that runs nothing, glog macros).
// `private` is lifted for this translation unit so that the private members can be driven
// with host tensors the caller fills, the way Detector::Detect (:275-295) drives them after
// its read-back.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <functional>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include <opencv2/opencv.hpp>

#define private public
#include "opengl/examples/ssd/detector.h"
#undef private
#include "opengl/examples/ssd/detector.cc"
#include "opengl/examples/ssd/common.cc"

void softmax(float* data_in, float* data_out, int num);

extern "C" {

// boxes [A,4] decoded corner boxes, logits [A,C]. Runs GenerateBoxInfo -> GetTopK -> NMS of the
// reference and writes the survivors in its order: rect (x, y, width, height), score, class.
// Returns their number (at most top_k).
int ogle_ref_detect(const float* boxes, const float* logits, int A, int C, int image_w, int image_h, float score_thr,
                    int top_k, float nms_thr, int* out_rect, float* out_score, int* out_class) {
    opengl::DetectorOptions options;
    options.model_name = "";
    options.input_width = image_w;
    options.input_height = image_h;
    options.topk = top_k;
    options.nms_threshold = nms_thr;
    options.score_threshold = score_thr;
    options.variances = {0.1f, 0.1f, 0.2f, 0.2f};
    options.input_names = {"input"};
    options.output_names = {"cls_logits", "box_preds", "anchors"};
    opengl::Detector det(options);
    // what LoadToOutputTensors (:242-273) leaves behind: [0] boxes, [1] class logits, on the host
    opengl::Tensor* b = opengl::Tensor::Empty(opengl::Tensor::DT_FLOAT, {1, A, 4}, dlxnet::TensorProto::ANY);
    opengl::Tensor* l = opengl::Tensor::Empty(opengl::Tensor::DT_FLOAT, {1, A, C}, dlxnet::TensorProto::ANY);
    std::memcpy(b->host<float>(), boxes, sizeof(float) * size_t(A) * 4);
    std::memcpy(l->host<float>(), logits, sizeof(float) * size_t(A) * C);
    det.output_tensors_ = {b, l};                      // the detector's destructor frees them
    det.origin_input_sizes_ = {image_h, image_w};      // Preprocess (:102) records rows, cols of the frame
    std::vector<BoxInfo> candidates, kept;
    det.GenerateBoxInfo(candidates, det.score_threshold_);
    det.GetTopK(candidates, det.topk_);
    det.NMS(candidates, kept, det.nms_threshold_);
    for (size_t i = 0; i < kept.size(); ++i) {
        out_rect[i * 4 + 0] = kept[i].box.x; out_rect[i * 4 + 1] = kept[i].box.y;
        out_rect[i * 4 + 2] = kept[i].box.width; out_rect[i * 4 + 3] = kept[i].box.height;
        out_score[i] = kept[i].score;
        out_class[i] = int(kept[i].class_name);
    }
    return int(kept.size());
}

// common.cc:86-97 on one row of n logits.
int ogle_ref_softmax(const float* in, float* out, int n) {
    std::vector<float> tmp(in, in + n);
    softmax(tmp.data(), out, n);
    return 0;
}

}  // extern "C"

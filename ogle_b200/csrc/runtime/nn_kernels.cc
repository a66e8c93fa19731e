// The operator kernels: one class per reference kernel under
// ogl_runtime/opengl/nn/kernels/, registered under the same ONNX operator names.
// Attribute parsing, variant selection, shape inference and the checks follow
// the reference; Compute calls include/ogle_cuda.h instead of drawing.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "fbo_session.h"
#include "kernel.h"
#include "kernel_registry.h"
#include "ogle_cuda.h"

namespace ogle {
namespace {

using TP = dlxnet::TensorProto;

bool IsPadded4(const Tensor* t) { return t->dformat() == TP::NHWC4 || t->dformat() == TP::ANY4; }

IntList AmendShape(const IntList& shape) {
    // left-pad to 4-D with 1s (ogl_runtime/opengl/utils/util.cc:44-59)
    OGLE_CHECK_LE(shape.size(), 4u);
    IntList s(4 - shape.size(), 1);
    s.insert(s.end(), shape.begin(), shape.end());
    return s;
}

long Rows(const Tensor* t) { return t->shape().empty() ? 1 : long(t->num_elements() / size_t(t->last_stride())); }

// Square kernel / equal strides / four equal pads, as conv2d.cc:67-88 and pool.cc:38-54.
void ParseWindow(const std::vector<int64_t>& kernel_shape, const std::vector<int64_t>& strides,
                 const std::vector<int64_t>& pads, int* kernel, int* stride, int* pad) {
    OGLE_CHECK_EQ(pads.size(), 4u);
    for (int64_t p : pads) OGLE_CHECK_EQ(pads[0], p);
    *pad = int(pads[0]);
    OGLE_CHECK_EQ(strides.size(), 2u);
    OGLE_CHECK_EQ(strides[0], strides[1]);
    *stride = int(strides[0]);
    OGLE_CHECK_EQ(kernel_shape.size(), 2u);
    OGLE_CHECK_EQ(kernel_shape[0], kernel_shape[1]);
    *kernel = int(kernel_shape[0]);
}

// ------------------------------------------------------------------- Const
// nn/kernels/const.cc:7-66
class ConstKernel : public Kernel {
public:
    explicit ConstKernel(Context* c) : Kernel(c) {}
    void SetupAttr(const dlxnet::Attribute& attr) override {
        OGLE_CHECK(!tensor_);
        tensor_.reset(new Tensor(attr.const_attr.value));
        output_tensor_dformats_.push_back(attr.const_attr.value.target_data_format);
        kernel_fname_ = "upload";
    }
    void Compute(TensorList& inputs, TensorList& outputs) override {
        OGLE_CHECK(inputs.empty()) << "Input should be empty in ConstKernel";
        context_->CopyCPUTensorToDevice(tensor_.get(), outputs[0]);
    }
    void InferOutputShape(TensorShapeList& inputs, TensorShapeList& outputs) override {
        OGLE_CHECK(inputs.empty()) << "Input should be empty in ConstKernel";
        const DataFormat f = output_tensor_dformats_[0];
        OGLE_CHECK(f == TP::ANY4 || f == TP::HWN4C4) << "unsupported dformat " << int(f) << " in Const Kernel " << kernel_name_;
        outputs.push_back(tensor_->shape());
    }
private:
    std::unique_ptr<Tensor> tensor_;
};
REGISTER_KERNEL_WITH_NAME(ConstKernel, "Const");
REGISTER_KERNEL_WITH_NAME(ConstKernel, "Constant");

// -------------------------------------------------------------------- Conv
// nn/kernels/conv2d.cc:19-197
class Conv2DKernel : public Kernel {
public:
    explicit Conv2DKernel(Context* c) : Kernel(c) {}
    ~Conv2DKernel() override {
        if (workspace_) cudaFree(workspace_);
        if (packed_) cudaFree(packed_);
        if (pair_packed_) cudaFree(pair_packed_);
        if (pair_bias_) cudaFree(pair_bias_);
    }

    void SetupAttr(const dlxnet::Attribute& attr) override {
        const auto& p = attr.conv2d_attr;
        ParseWindow(p.kernel_shape, p.strides, p.pads, &kernel_size_, &stride_, &padding_);
        group_size_ = int(p.group);
        if (group_size_ == 0) group_size_ = 1;
        if (p.dilations.size() == 2) {
            OGLE_CHECK_EQ(p.dilations[0], p.dilations[1]);
            dilation_ = int(p.dilations[0]);
        } else if (p.dilations.size() == 1) {
            dilation_ = int(p.dilations[0]);
        } else {
            dilation_ = 1;
        }
        activation_type_ = p.activation_type;
        min_ = p.min;
        max_ = p.max;
    }

    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(inputs.size() == 2 || inputs.size() == 3);
        OGLE_CHECK(IsPadded4(inputs[0])) << "conv input must be NHWC4 or ANY4";
        OGLE_CHECK_EQ(inputs[0]->shape().size(), 4u);
        const bool pw = kernel_size_ == 1 && group_size_ == 1 && dilation_ == 1 && stride_ == 1 && padding_ == 0;
        if (pw) kernel_fname_ = "conv2d_pw";
        else if (group_size_ != 1)
            kernel_fname_ = (group_size_ == inputs[0]->shape()[3] && group_size_ == inputs[1]->shape()[0]) ? "conv2d_dw" : "conv2d_grp";
        else kernel_fname_ = "conv2d";
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }

    void InferOutputShape(const TensorList& inputs, TensorShapeList& output_shapes) override {
        Kernel::InferOutputShape(inputs, output_shapes);
        // the filter is re-laid out once when it is a model constant (the reference does
        // this in its upload pass); otherwise before every launch
        const size_t bytes = ogle_cuda_conv2d_filter_bytes(&params_);
        OGLE_CHECK_GT(bytes, 0u);
        if (packed_) cudaFree(packed_);
        cudaError_t e = cudaMalloc(&packed_, bytes);
        OGLE_CHECK(e == cudaSuccess) << "cudaMalloc(" << bytes << "): " << cudaGetErrorString(e);
        filter_is_constant_ = session_ && session_->IsTensorReady(input_tensor_indexes_[1]);
        if (filter_is_constant_)
            OGLE_CUDA_OK(ogle_cuda_conv2d_prepack(&params_, inputs[1]->device<float>(), packed_, context_->stream()));
        EnsureWorkspace(ogle_cuda_conv2d_workspace_bytes(&params_));
    }

    // Scratch for layers that split their reduction (long reductions over few tiles): allocated with the
    // tensors, never in steady state.
    void EnsureWorkspace(size_t bytes) {
        if (bytes <= workspace_bytes_) return;
        if (workspace_) cudaFree(workspace_);
        workspace_ = nullptr;
        workspace_bytes_ = 0;
        cudaError_t e = cudaMalloc(&workspace_, bytes);
        OGLE_CHECK(e == cudaSuccess) << "cudaMalloc(" << bytes << "): " << cudaGetErrorString(e);
        workspace_bytes_ = bytes;
    }

    void InferOutputShape(TensorShapeList& input_shapes, TensorShapeList& output_shapes) override {
        OGLE_CHECK(input_shapes.size() == 3 || input_shapes.size() == 2);
        output_shapes.clear();
        output_shapes.resize(1);
        const IntList& image_shape = input_shapes[0];
        const IntList& filter_shape = input_shapes[1];
        OGLE_CHECK_EQ(image_shape.size(), 4u);
        OGLE_CHECK_EQ(filter_shape.size(), 4u);
        OGLE_CHECK_EQ(filter_shape[2], kernel_size_);
        OGLE_CHECK_EQ(filter_shape[3], kernel_size_);
        OGLE_CHECK_EQ(filter_shape[1] * group_size_, image_shape[3]);
        std::memset(&params_, 0, sizeof(params_));
        params_.N = image_shape[0];
        params_.in_hwc[0] = image_shape[1]; params_.in_hwc[1] = image_shape[2]; params_.in_hwc[2] = image_shape[3];
        params_.out_hwc[2] = filter_shape[0];
        params_.kernel = kernel_size_; params_.stride = stride_; params_.pad = padding_;
        params_.dilation = dilation_; params_.group = group_size_;
        params_.has_bias = input_shapes.size() > 2;
        params_.act = activation_type_ == "Clip" ? OGLE_ACT_CLIP : (activation_type_ == "Relu" ? OGLE_ACT_RELU : OGLE_ACT_NONE);
        if (!activation_type_.empty() && params_.act == OGLE_ACT_NONE) params_.act = OGLE_ACT_RELU;  // conv2d.cc:137-143
        params_.min_value = min_; params_.max_value = max_;
        params_.math_mode = context_->math_mode();
        OGLE_CUDA_OK(ogle_cuda_conv2d_infer(&params_));
        // family (the reference's shader name) : device kernel that serves it
        const size_t colon = kernel_fname_.find(':');
        kernel_fname_ = kernel_fname_.substr(0, colon) + ":" + ogle_cuda_conv2d_kernel_name(&params_);
        output_shapes[0] = {image_shape[0], params_.out_hwc[0], params_.out_hwc[1], filter_shape[0]};
    }

    // Two convolutions over one feature map with the same window and constant filters run as
    // one pass: the filters are stacked (first conv's rows, zero rows up to a multiple of 32,
    // second conv's rows) and packed once; Compute then writes both nodes' outputs.
    bool AbsorbSibling(Kernel* later) override {
        auto* o = dynamic_cast<Conv2DKernel*>(later);
        if (!o || o == this || sibling_ || o->sibling_) return false;
        if (!filter_is_constant_ || !o->filter_is_constant_) return false;
        if (input_tensors_.size() != o->input_tensors_.size() || input_tensors_[0] != o->input_tensors_[0]) return false;
        const OgleConvParams &a = params_, &b = o->params_;
        if (a.group != 1 || b.group != 1 || a.kernel != b.kernel || a.stride != b.stride || a.pad != b.pad ||
            a.dilation != b.dilation || a.act != b.act || a.min_value != b.min_value || a.max_value != b.max_value ||
            a.math_mode != b.math_mode || a.has_bias != b.has_bias)
            return false;
        if (a.has_bias && !(session_->IsTensorReady(input_tensor_indexes_[2]) && session_->IsTensorReady(o->input_tensor_indexes_[2])))
            return false;
        const int K1 = a.out_hwc[2], K2 = b.out_hwc[2], split = (K1 + 31) / 32 * 32;
        OgleConvParams f = a;
        f.out_hwc[2] = split + K2;
        if (!ogle_cuda_conv2d_pair_supported(&f)) return false;
        cudaStream_t s = reinterpret_cast<cudaStream_t>(context_->stream());
        const size_t row = size_t(a.in_hwc[2]) * a.kernel * a.kernel;      // floats per output channel (OIHW)
        float* stacked = nullptr;
        auto ok = [](cudaError_t e) { OGLE_CHECK(e == cudaSuccess) << "sibling fusion: " << cudaGetErrorString(e); };
        ok(cudaMalloc(&stacked, size_t(split + K2) * row * 4));
        ok(cudaMemsetAsync(stacked, 0, size_t(split + K2) * row * 4, s));
        ok(cudaMemcpyAsync(stacked, input_tensors_[1]->device<float>(), size_t(K1) * row * 4, cudaMemcpyDeviceToDevice, s));
        ok(cudaMemcpyAsync(stacked + size_t(split) * row, o->input_tensors_[1]->device<float>(), size_t(K2) * row * 4,
                           cudaMemcpyDeviceToDevice, s));
        const size_t bytes = ogle_cuda_conv2d_filter_bytes(&f);
        OGLE_CHECK_GT(bytes, 0u);
        ok(cudaMalloc(&pair_packed_, bytes));
        OGLE_CUDA_OK(ogle_cuda_conv2d_prepack(&f, stacked, pair_packed_, context_->stream()));
        if (a.has_bias) {
            ok(cudaMalloc(&pair_bias_, size_t(split + K2 + 4) * 4));
            ok(cudaMemsetAsync(pair_bias_, 0, size_t(split + K2 + 4) * 4, s));
            ok(cudaMemcpyAsync(pair_bias_, input_tensors_[2]->device<float>(), size_t(K1) * 4, cudaMemcpyDeviceToDevice, s));
            ok(cudaMemcpyAsync(pair_bias_ + split, o->input_tensors_[2]->device<float>(), size_t(K2) * 4, cudaMemcpyDeviceToDevice, s));
        }
        ok(cudaStreamSynchronize(s));
        cudaFree(stacked);
        pair_params_ = f;
        pair_k1_ = K1;
        pair_split_ = split;
        EnsureWorkspace(ogle_cuda_conv2d_pair_workspace_bytes(&f, K1, split));
        sibling_ = o;
        kernel_name_ += "+" + o->kernel_name_;
        return true;
    }

    // Channel-axis concat in place: the pixels of this conv are the rows, its channels the chunk
    // (the out_channel_offset / out_channel_stride fields of the conv call; replaces one
    // copy pass of concat.cc:73-96).
    bool PlaceOutput(Tensor* dst, long outer, long chunk, long row_stride, long offset) override {
        if (sibling_ || placed_ || output_tensors_.empty()) return false;
        const long pixels = long(params_.N) * params_.out_hwc[0] * params_.out_hwc[1];
        if (outer != pixels || chunk != UpRound4(params_.out_hwc[2]) || (row_stride & 3) || (offset & 3)) return false;
        if (offset + chunk > row_stride || params_.out_channel_stride || params_.out_channel_offset) return false;
        OgleConvParams q = params_;
        q.out_channel_stride = int(row_stride);
        q.out_channel_offset = int(offset);
        if (ogle_cuda_conv2d_infer(&q) != OGLE_OK) return false;
        params_ = q;
        placed_ = dst;
        const size_t colon = kernel_fname_.find(':');
        kernel_fname_ = kernel_fname_.substr(0, colon) + ":" + ogle_cuda_conv2d_kernel_name(&params_);
        return true;
    }

    // A residual block's tail: y = act(conv(x) + bias + residual) in the convolution's pass
    // (ogle_cuda_conv2d_residual; same fp32 operations in the same order as conv, binary add and activation
    // passes, nn/kernels/binary.cc + relu.cc). Relu or no activation only: a Clip keeps its own pass, because a
    // pointwise convolution's built-in clip clamps to [0, max] (conv2d_pw.glsl:85), not to [min, max].
    bool AbsorbResidualAdd(Kernel* add, Tensor* residual, Tensor* dst, int act, float lo, float hi) override {
        if (sibling_ || placed_ || residual_ || !filter_is_constant_ || output_tensors_.empty()) return false;
        if (params_.act != OGLE_ACT_NONE || (act != OGLE_ACT_NONE && act != OGLE_ACT_RELU)) return false;
        if (params_.out_channel_stride || params_.out_channel_offset) return false;
        if (!ogle_cuda_conv2d_residual_supported(&params_)) return false;
        if (residual->AllocatedSize() != output_tensors_[0]->AllocatedSize() ||
            dst->AllocatedSize() != output_tensors_[0]->AllocatedSize())
            return false;
        params_.act = act;
        params_.min_value = lo;
        params_.max_value = hi;
        residual_ = residual;
        residual_dst_ = dst;
        kernel_name_ += "+" + add->kernel_name();
        return true;
    }

    // The tensor-core path's tile width (output channels per tile) decides how many tiles a layer has, how
    // deep its operand ring is and how long a tile's epilogue takes; which width wins depends on the batch
    // (rounds of tiles over the SMs) in ways a cost model only approximates. Every width gives the same bits,
    // so the layer simply times the candidates on its own tensors and keeps the fastest; then, at that width, the
    // number of ranges its reduction is split into (which does change the order of the partial sums); last, for
    // an unsplit reduction, whether pairs of SMs should share the filter tiles (same bits again).
    void Tune() override {
        OgleConvParams& p = sibling_ ? pair_params_ : params_;
        if (!filter_is_constant_ || std::string(ogle_cuda_conv2d_kernel_name(&p)) != "conv_tc2_kernel") return;
        cudaStream_t s = reinterpret_cast<cudaStream_t>(context_->stream());
        cudaEvent_t e0, e1;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return;
        const int kmax = (p.out_hwc[2] + 31) / 32 * 32;
        auto workspace_for = [&] {
            EnsureWorkspace(sibling_ ? ogle_cuda_conv2d_pair_workspace_bytes(&p, pair_k1_, pair_split_)
                                     : ogle_cuda_conv2d_workspace_bytes(&p));
        };
        auto time_it = [&](float* ms) {
            workspace_for();
            Kernel::Compute();                                          // warm-up
            cudaEventRecord(e0, s);
            for (int r = 0; r < 3; ++r) Kernel::Compute();
            cudaEventRecord(e1, s);
            if (cudaEventSynchronize(e1) != cudaSuccess) return false;
            return cudaEventElapsedTime(ms, e0, e1) == cudaSuccess;
        };
        float auto_ms = 0.f, best_ms = 0.f;
        p.n_tile = 0;
        p.split = 0;
        p.sm_pair = 0;
        p.channels_on_m = 0;
        if (time_it(&auto_ms)) {
            best_ms = auto_ms;
            int best_tile = 0, best_split = 0, best_pair = 0;
            for (int bn = 32; bn <= 256 && bn <= kmax; bn += 32) {          // tile widths, the library's split rule
                float ms;
                p.n_tile = bn;
                if (time_it(&ms) && ms < best_ms) { best_ms = ms; best_tile = bn; }
            }
            p.n_tile = best_tile;
            static const int splits[] = {1, 2, 3, 4, 6, 8, 12, 16};          // then the reduction split at that width
            for (int k : splits) {
                float ms;
                p.split = k;
                if (time_it(&ms) && ms < best_ms) { best_ms = ms; best_split = k; }
            }
            p.split = best_split;
            int pair_tile = best_tile;
            for (int bn = 64; bn <= 256 && bn <= kmax; bn += 64) {           // SM pairs, unsplit, at the widths that halve
                float ms;
                p.n_tile = bn;
                p.split = 1;
                p.sm_pair = 2;
                if (time_it(&ms) && ms < best_ms) { best_ms = ms; best_pair = 2; pair_tile = bn; }
            }
            if (best_pair) { best_tile = pair_tile; best_split = 1; }
            // at most 128 output channels: the accumulator kept transposed (filters on the multiply's 128-row side)
            int best_on_m = 0;
            if (p.out_hwc[2] <= 128) {
                float ms;
                p.n_tile = 0;
                p.split = 1;
                p.sm_pair = 1;
                p.channels_on_m = 2;
                if (time_it(&ms) && ms < best_ms) { best_ms = ms; best_on_m = 2; best_pair = 0; best_tile = 0; best_split = 1; }
                static const int t_splits[] = {2, 3, 4, 6, 8};          // and with the reduction split through scratch
                for (int k : t_splits) {
                    p.split = k;
                    if (time_it(&ms) && ms < best_ms) { best_ms = ms; best_on_m = 2; best_pair = 0; best_tile = 0; best_split = k; }
                }
                p.channels_on_m = 0;
            }
            if (best_ms > 0.97f * auto_ms) { best_tile = 0; best_split = 0; best_pair = 0; best_on_m = 0; }   // within noise of the defaults: keep them
            p.n_tile = best_tile;
            p.split = best_split;
            p.sm_pair = best_pair;
            p.channels_on_m = best_on_m;
            tuned_tile_ = best_tile;
            tuned_split_ = best_split;
            tuned_pair_ = best_pair;
        }
        workspace_for();
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    int tuned_tile() const { return tuned_tile_; }

    void Compute(TensorList& inputs, TensorList& outputs) override {
        if (sibling_) {
            OGLE_CUDA_OK(ogle_cuda_conv2d_pair_ws(&pair_params_, inputs[0]->device<float>(), pair_packed_, pair_bias_, pair_k1_,
                                                  pair_split_, outputs[0]->device<float>(),
                                                  sibling_->output_tensors_[0]->device<float>(), workspace_, workspace_bytes_,
                                                  context_->stream()));
            return;
        }
        if (!filter_is_constant_)
            OGLE_CUDA_OK(ogle_cuda_conv2d_prepack(&params_, inputs[1]->device<float>(), packed_, context_->stream()));
        const float* bias = inputs.size() > 2 ? inputs[2]->device<float>() : nullptr;
        if (residual_) {
            OGLE_CUDA_OK(ogle_cuda_conv2d_residual(&params_, inputs[0]->device<float>(), packed_, bias, residual_->device<float>(),
                                                   0, residual_dst_->device<float>(), context_->stream()));
            return;
        }
        float* y = placed_ ? placed_->device<float>() : outputs[0]->device<float>();
        OGLE_CUDA_OK(ogle_cuda_conv2d_ws(&params_, inputs[0]->device<float>(), packed_, bias, y, workspace_, workspace_bytes_,
                                         context_->stream()));
    }

private:
    int padding_ = 0, stride_ = 1, kernel_size_ = 1, group_size_ = 1, dilation_ = 1;
    std::string activation_type_;
    float min_ = 0.f, max_ = 0.f;
    OgleConvParams params_;
    void* packed_ = nullptr;
    void* workspace_ = nullptr;
    size_t workspace_bytes_ = 0;
    bool filter_is_constant_ = false;
    Conv2DKernel* sibling_ = nullptr;       // absorbed later node (not owned)
    Tensor* placed_ = nullptr;              // a concat's tensor this conv writes into (not owned)
    Tensor* residual_ = nullptr;            // a residual block's other operand, added in this conv's pass (not owned)
    Tensor* residual_dst_ = nullptr;        // where that sum (after the activation) goes (not owned)
    int tuned_tile_ = 0, tuned_split_ = 0, tuned_pair_ = 0;
    OgleConvParams pair_params_;
    void* pair_packed_ = nullptr;
    float* pair_bias_ = nullptr;
    int pair_k1_ = 0, pair_split_ = 0;
};
REGISTER_KERNEL_WITH_NAME(Conv2DKernel, "Conv");

// ------------------------------------------------------ BatchNormalization
// nn/kernels/batchnorm.cc:14-95
class BatchNormKernel : public Kernel {
public:
    explicit BatchNormKernel(Context* c) : Kernel(c) { kernel_fname_ = "batchnorm"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        momentum_ = attr.batchnorm_attr.momentum;
        eps_ = attr.batchnorm_attr.epsilon;
    }
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 5u);
        for (int i = 1; i < 5; ++i) {
            OGLE_CHECK_EQ(in[i].size(), 1u);
            OGLE_CHECK_EQ(in[i][0], in[0].back());
        }
        out.assign(1, in[0]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CUDA_OK(ogle_cuda_batchnorm(in[0]->device<float>(), in[1]->device<float>(), in[2]->device<float>(),
                                         in[3]->device<float>(), in[4]->device<float>(), out[0]->device<float>(),
                                         Rows(in[0]), in[0]->last_stride(), 0, eps_, context_->stream()));
    }
private:
    float momentum_ = 0.f, eps_ = 0.f;
};
REGISTER_KERNEL_WITH_NAME(BatchNormKernel, "BatchNormalization");

// ------------------------------------------------------- Relu / Clip / Add
// nn/kernels/relu.cc, clip.cc, binary.cc
class ReluKernel : public Kernel {
public:
    explicit ReluKernel(Context* c) : Kernel(c) { kernel_fname_ = "relu"; }
    void SetupAttr(const dlxnet::Attribute&) override {}
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        out.assign(1, in[0]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CUDA_OK(ogle_cuda_relu(in[0]->device<float>(), out[0]->device<float>(), long(in[0]->AllocatedElements()),
                                    context_->stream()));
    }
    bool AsActivation(int* act, float* lo, float* hi) const override {
        *act = OGLE_ACT_RELU; *lo = 0.f; *hi = 0.f;
        return true;
    }
};
REGISTER_KERNEL_WITH_NAME(ReluKernel, "Relu");

class ClipKernel : public Kernel {
public:
    explicit ClipKernel(Context* c) : Kernel(c) { kernel_fname_ = "clip"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        min_ = attr.clip_attr.min;
        max_ = attr.clip_attr.max;
    }
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        out.assign(1, in[0]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CUDA_OK(ogle_cuda_clip(in[0]->device<float>(), out[0]->device<float>(), long(in[0]->AllocatedElements()),
                                    min_, max_, context_->stream()));
    }
    bool AsActivation(int* act, float* lo, float* hi) const override {
        *act = OGLE_ACT_CLIP; *lo = min_; *hi = max_;
        return true;
    }
private:
    float min_ = 0.f, max_ = 0.f;
};
REGISTER_KERNEL_WITH_NAME(ClipKernel, "Clip");

class BinaryKernel : public Kernel {
public:
    explicit BinaryKernel(Context* c) : Kernel(c) { kernel_fname_ = "binary_add"; }
    void SetupAttr(const dlxnet::Attribute&) override {}
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        // same-shape operands only; the reference has no broadcast (binary.cc:55-63)
        OGLE_CHECK_EQ(in.size(), 2u);
        OGLE_CHECK_EQ(in[0].size(), in[1].size());
        for (size_t i = 0; i < in[0].size(); ++i) OGLE_CHECK_EQ(in[0][i], in[1][i]);
        out.assign(1, in[0]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        float* y = act_out_ ? act_out_->device<float>() : out[0]->device<float>();
        OGLE_CUDA_OK(ogle_cuda_add_act(in[0]->device<float>(), in[1]->device<float>(), y, long(in[0]->AllocatedElements()),
                                       act_, act_lo_, act_hi_, context_->stream()));
    }
    bool AsResidualAdd(int* act, float* lo, float* hi, Tensor** dst) const override {
        if (output_tensors_.empty()) return false;
        *act = act_; *lo = act_lo_; *hi = act_hi_;
        *dst = act_out_ ? act_out_ : output_tensors_[0];
        return true;
    }
    // a residual block's Add -> Relu (or Clip) as one pass
    bool AbsorbConsumer(Kernel* consumer) override {
        if (act_out_ || consumer == this) return false;
        int act; float lo, hi;
        if (!consumer->AsActivation(&act, &lo, &hi)) return false;
        const TensorList& co = ConsumerOutputs(consumer);
        if (co.size() != 1 || co[0]->AllocatedSize() != output_tensors_[0]->AllocatedSize()) return false;
        act_ = act; act_lo_ = lo; act_hi_ = hi;
        act_out_ = co[0];
        kernel_fname_ = act == OGLE_ACT_RELU ? "binary_add_relu" : "binary_add_clip";
        kernel_name_ += "+" + consumer->kernel_name();
        return true;
    }
private:
    int act_ = OGLE_ACT_NONE;
    float act_lo_ = 0.f, act_hi_ = 0.f;
    Tensor* act_out_ = nullptr;      // the absorbed activation's output; not owned
};
REGISTER_KERNEL_WITH_NAME(BinaryKernel, "Add");

// -------------------------------------------------------------------- Pool
// nn/kernels/pool.cc:26-129
enum PoolType { MaxPool = 0, AveragePool = 1, GlobalAveragePool = 2 };
template <PoolType pool_type>
class PoolKernel : public Kernel {
public:
    explicit PoolKernel(Context* c) : Kernel(c) { kernel_fname_ = pool_type == MaxPool ? "pool_max" : "pool_avg"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        if (pool_type == GlobalAveragePool) return;
        // both MaxPool and AveragePool read maxpool_attr (pool.cc:32)
        const auto& p = attr.maxpool_attr;
        ParseWindow(p.kernel_shape, p.strides, p.pads, &kernel_size_, &stride_, &padding_);
    }
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(inputs[0]->dformat());
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        OGLE_CHECK_EQ(in[0].size(), 4u);
        std::memset(&params_, 0, sizeof(params_));
        params_.N = in[0][0];
        params_.in_hwc[0] = in[0][1]; params_.in_hwc[1] = in[0][2]; params_.in_hwc[2] = in[0][3];
        params_.kernel = kernel_size_; params_.stride = stride_; params_.pad = padding_;
        params_.type = int(pool_type);
        if (pool_type == GlobalAveragePool) { OGLE_CHECK_EQ(in[0][1], in[0][2]); }  // pool.cc:88
        OGLE_CUDA_OK(ogle_cuda_pool_infer(&params_));
        out.assign(1, IntList{in[0][0], params_.out_hwc[0], params_.out_hwc[1], in[0][3]});
    }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CUDA_OK(ogle_cuda_pool(&params_, in[0]->device<float>(), out[0]->device<float>(), context_->stream()));
    }
private:
    int kernel_size_ = 1, stride_ = 1, padding_ = 0;
    OglePoolParams params_;
};
REGISTER_KERNEL_WITH_NAME(PoolKernel<MaxPool>, "MaxPool");
REGISTER_KERNEL_WITH_NAME(PoolKernel<AveragePool>, "AveragePool");
REGISTER_KERNEL_WITH_NAME(PoolKernel<GlobalAveragePool>, "GlobalAveragePool");

// -------------------------------------------------------------------- Gemm
// nn/kernels/gemm.cc:16-108
class GemmKernel : public Kernel {
public:
    explicit GemmKernel(Context* c) : Kernel(c) { kernel_fname_ = "gemm"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        alpha_ = attr.gemm_attr.alpha;
        beta_ = attr.gemm_attr.beta;
        transB_ = attr.gemm_attr.transb;
        output_tensor_dformats_.push_back(TP::ANY4);
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        out.clear();
        out.resize(1);
        OGLE_CHECK_GE(in.size(), 2u);
        OGLE_CHECK_EQ(in[0].size(), 2u);
        OGLE_CHECK_EQ(in[1].size(), 2u);
        if (transB_) {
            OGLE_CHECK_EQ(in[1][1], in[0][1]);
            out[0] = {in[0][0], in[1][0]};
        } else {
            OGLE_CHECK_EQ(in[1][0], in[0][1]);
            out[0] = {in[0][0], in[1][1]};
        }
        std::memset(&params_, 0, sizeof(params_));
        params_.M = out[0][0]; params_.K = in[0][1]; params_.N = out[0][1];
        params_.transB = transB_; params_.alpha = alpha_; params_.beta = beta_;
        params_.math_mode = context_->math_mode();
        if (in.size() > 2) {
            if (in[2].size() == 2) {
                OGLE_CHECK_EQ(out[0][0], in[2][0]);
                OGLE_CHECK_EQ(out[0][1], in[2][1]);
                params_.bias_mode = 1;
            } else {
                // a [N] bias is broadcast over rows (ONNX); the reference's shader is
                // only correct for M == 1 here (gemm.glsl:92-94)
                OGLE_CHECK_EQ(in[2].size(), 1u);
                OGLE_CHECK_EQ(out[0][1], in[2][0]);
                params_.bias_mode = 2;
            }
        }
    }
    void InferOutputShape(const TensorList& inputs, TensorShapeList& output_shapes) override {
        Kernel::InferOutputShape(inputs, output_shapes);
        // constant weights are re-laid once for the tensor-core modes, as conv filters are
        packed_ready_ = false;
        if (params_.math_mode != OGLE_MATH_FP32 && session_ && session_->IsTensorReady(input_tensor_indexes_[1]) &&
            params_.K >= 64) {
            const size_t bytes = ogle_cuda_gemm_packed_b_bytes(&params_);
            OGLE_CHECK_GT(bytes, 0u);
            if (packed_) cudaFree(packed_);
            cudaError_t e = cudaMalloc(&packed_, bytes);
            OGLE_CHECK(e == cudaSuccess) << "cudaMalloc(" << bytes << "): " << cudaGetErrorString(e);
            OGLE_CUDA_OK(ogle_cuda_gemm_pack_b(&params_, inputs[1]->device<float>(), packed_, context_->stream()));
            packed_ready_ = true;
        }
    }
    ~GemmKernel() override { if (packed_) cudaFree(packed_); }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CHECK_EQ(in[0]->dformat(), TP::ANY4);
        OGLE_CHECK_EQ(in[1]->dformat(), TP::ANY4);
        const float* c = in.size() > 2 ? in[2]->device<float>() : nullptr;
        if (packed_ready_) {
            OGLE_CUDA_OK(ogle_cuda_gemm_packed(&params_, in[0]->device<float>(), packed_, c, out[0]->device<float>(),
                                               context_->stream()));
            return;
        }
        OGLE_CUDA_OK(ogle_cuda_gemm(&params_, in[0]->device<float>(), in[1]->device<float>(), c, out[0]->device<float>(),
                                    context_->stream()));
    }
private:
    float alpha_ = 1.f, beta_ = 1.f;
    int transB_ = 0;
    OgleGemmParams params_;
    void* packed_ = nullptr;
    bool packed_ready_ = false;
};
REGISTER_KERNEL_WITH_NAME(GemmKernel, "Gemm");

// ------------------------------------------------------------------ Concat
// nn/kernels/concat.cc:32-133
class ConcatKernel : public Kernel {
public:
    explicit ConcatKernel(Context* c) : Kernel(c) { kernel_fname_ = "concat"; }
    void SetupAttr(const dlxnet::Attribute& attr) override { axis_ = attr.concat_attr.axis; }
    void SelectKernel(const TensorList& inputs) override {
        // The reference accepts ANY4 inputs only (concat.cc:33). NHWC4 has the same
        // bytes in linear memory, so it is accepted too, with the ONNX (NCHW) axis
        // mapped onto the stored NHWC order as concat.cc:42-45 does.
        for (auto t : inputs) OGLE_CHECK(IsPadded4(t)) << "concat inputs must be ANY4 or NHWC4";
        output_tensor_dformats_.push_back(TP::ANY4);
        if (session_ && session_->IsONNX() && inputs[0]->dformat() == TP::NHWC4 && axis_ >= 0) {
            static const int mapping[4] = {0, 3, 1, 2};
            OGLE_CHECK_LT(axis_, 4);
            axis_ = mapping[axis_];
        }
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        if (axis_ < 0) axis_ += int(in[0].size());   // concat.cc:101-103 handles -1
        OGLE_CHECK_GE(in.size(), 2u);
        OGLE_CHECK_LE(in.size(), size_t(OGLE_MAX_CONCAT_INPUTS));
        OGLE_CHECK(axis_ >= 0 && axis_ < int(in[0].size()));
        out.assign(1, in[0]);
        out[0][axis_] = 0;
        for (auto& s : in) {
            OGLE_CHECK_EQ(out[0].size(), s.size());
            for (size_t i = 0; i < s.size(); ++i) {
                if (int(i) != axis_) OGLE_CHECK_EQ(s[i], out[0][i]);
                else out[0][i] += s[i];
            }
        }
        std::memset(&params_, 0, sizeof(params_));
        params_.n_inputs = int(in.size());
        params_.axis = axis_ + 4 - int(in[0].size());   // concat.cc:61
        for (size_t i = 0; i < in.size(); ++i) {
            const IntList s4 = AmendShape(in[i]);
            for (int d = 0; d < 4; ++d) params_.in_shapes[i][d] = s4[d];
        }
    }
    void Compute(TensorList& in, TensorList& out) override {
        const float* ptrs[OGLE_MAX_CONCAT_INPUTS];
        for (size_t i = 0; i < in.size(); ++i) ptrs[i] = (placed_mask_ >> i) & 1u ? nullptr : in[i]->device<float>();
        OGLE_CUDA_OK(ogle_cuda_concat(&params_, ptrs, out[0]->device<float>(), context_->stream()));
    }
    bool ConcatPlacement(int input, long* outer, long* chunk, long* row_stride, long* offset) const override {
        const int n = params_.n_inputs, a = params_.axis;
        if (input < 0 || input >= n) return false;
        long before = 1, inner = 1, start = 0, total = 0;
        for (int d = 0; d < a; ++d) before *= params_.in_shapes[0][d];
        for (int d = a + 1; d < 4; ++d) inner *= d == 3 ? UpRound4(params_.in_shapes[0][3]) : params_.in_shapes[0][d];
        for (int i = 0; i < n; ++i) {
            if (i == input) start = total;
            total += params_.in_shapes[i][a];
        }
        const long extent = params_.in_shapes[input][a];
        if (a == 3) {
            // slices start on a multiple of four channels; only the last may end off one
            if ((start & 3) || ((extent & 3) && input + 1 < n)) return false;
            *chunk = UpRound4(int(extent)); *row_stride = UpRound4(int(total)); *offset = start;
        } else {
            *chunk = extent * inner; *row_stride = total * inner; *offset = start * inner;
        }
        *outer = before;
        return true;
    }
    void InputPlaced(int input) override { placed_mask_ |= 1u << input; }
private:
    int axis_ = 0;
    unsigned placed_mask_ = 0;
    OgleConcatParams params_;
};
REGISTER_KERNEL_WITH_NAME(ConcatKernel, "Concat");

// --------------------------------------------------------------- Transpose
// nn/kernels/transpose.cc:34-105
class TransposeKernel : public Kernel {
public:
    explicit TransposeKernel(Context* c) : Kernel(c) { kernel_fname_ = "transpose"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        for (int p : attr.transpose_attr.perm) perm_.push_back(p);
    }
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(TP::ANY4);
        if (session_ && session_->IsONNX() && inputs[0]->dformat() == TP::NHWC4) {
            // the stored order is NHWC while perm is in ONNX (NCHW) terms
            OGLE_CHECK_EQ(perm_.size(), 4u);
            static const int mapping[4] = {0, 3, 1, 2};
            for (int& p : perm_) p = mapping[p];
        }
        identity_ = true;
        for (size_t i = 0; i < perm_.size(); ++i) identity_ = identity_ && perm_[i] == int(i);
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        OGLE_CHECK_LE(perm_.size(), in[0].size());
        out.assign(1, IntList());
        for (int p : perm_) out[0].push_back(in[0][p]);
        for (size_t i = perm_.size(); i < in[0].size(); ++i) out[0].push_back(in[0][i]);
        in_shape4_ = AmendShape(in[0]);
        // AmendPerm, transpose.cc:12-21
        perm4_.clear();
        for (size_t i = 0; i < 4 - perm_.size(); ++i) perm4_.push_back(int(i));
        for (int p : perm_) perm4_.push_back(p + 4 - int(perm_.size()));
    }
    bool IsNoOp() const override { return identity_; }
    void Compute(TensorList& in, TensorList& out) override {
        if (identity_) return;
        OGLE_CUDA_OK(ogle_cuda_transpose(in[0]->device<float>(), out[0]->device<float>(), in_shape4_.data(), perm4_.data(),
                                         context_->stream()));
    }
private:
    IntList perm_, perm4_, in_shape4_;
    bool identity_ = false;
};
REGISTER_KERNEL_WITH_NAME(TransposeKernel, "Transpose");

// ----------------------------------------------------------------- Reshape
// nn/kernels/reshape.cc:18-97
class ReshapeKernel : public Kernel {
public:
    explicit ReshapeKernel(Context* c) : Kernel(c) { kernel_fname_ = "reshape"; }
    void SetupAttr(const dlxnet::Attribute&) override {}
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        output_tensor_dformats_.push_back(TP::ANY4);
    }
    void InferOutputShape(TensorShapeList&, TensorShapeList&) override {
        OGLE_FATAL() << "Reshape needs the value of its shape input";
    }
    void InferOutputShape(const TensorList& inputs, TensorShapeList& out) override {
        out.clear();
        out.resize(1);
        OGLE_CHECK_EQ(inputs.size(), 2u);
        // the target shape is a (float-valued) device tensor computed at setup
        Tensor cpu(Tensor::DT_FLOAT, inputs[1]->shape(), Tensor::HOST_MEMORY, TP::ANY);
        context_->CopyDeviceTensorToCPU(inputs[1], &cpu);
        IntList& shape = out[0];
        for (size_t i = 0; i < cpu.num_elements(); ++i) shape.push_back(int(std::lround(cpu.host<float>()[i])));
        const IntList& in_shape = inputs[0]->shape();
        const long n = long(inputs[0]->num_elements());
        long remain = 1;
        for (size_t i = 0; i < shape.size(); ++i) {
            if (shape[i] == 0) {
                OGLE_CHECK_LT(i, in_shape.size());
                shape[i] = in_shape[i];
            }
            if (shape[i] != -1) remain *= shape[i];
        }
        bool seen = false;
        for (int& d : shape) {
            if (d == -1) {
                OGLE_CHECK(!seen) << "more than one -1 in a reshape target";
                OGLE_CHECK(remain > 0 && n % remain == 0);
                d = int(n / remain);
                seen = true;
            }
        }
        long total = 1;
        for (int d : shape) total *= d;
        OGLE_CHECK_EQ(total, n) << "reshape changes the element count";
        OGLE_CHECK_LE(shape.size(), 4u);
        n_ = n;
        in_last_ = inputs[0]->last_stride();
        out_last_ = shape.empty() ? 1 : shape.back();
        // same bytes when neither side pads, or the padded row is unchanged
        alias_ = (in_last_ == out_last_) || (in_last_ % 4 == 0 && out_last_ % 4 == 0);
    }
    bool IsNoOp() const override { return alias_; }
    void Compute(TensorList& in, TensorList& out) override {
        if (alias_) return;
        if (placed_) {
            OGLE_CUDA_OK(ogle_cuda_reshape_placed(in[0]->device<float>(), placed_->device<float>() + place_offset_, n_, in_last_,
                                                  out_last_, rows_per_block_, block_stride_, context_->stream()));
            return;
        }
        OGLE_CUDA_OK(ogle_cuda_reshape(in[0]->device<float>(), out[0]->device<float>(), n_, in_last_, out_last_,
                                       context_->stream()));
    }
    // The re-padding copy writes its rows where the concat wants them (the SSD class heads:
    // [N, h*w*a, C] slices of [N, anchors, C]).
    bool PlaceOutput(Tensor* dst, long outer, long chunk, long row_stride, long offset) override {
        if (alias_ || placed_) return false;
        const long row = UpRound4(out_last_);
        const long rows = n_ / out_last_;
        if (chunk % row || outer <= 0 || rows % outer || rows / outer != chunk / row || (row_stride & 3) || (offset & 3))
            return false;
        placed_ = dst; place_offset_ = offset; rows_per_block_ = chunk / row; block_stride_ = row_stride;
        return true;
    }
private:
    long n_ = 0;
    int in_last_ = 1, out_last_ = 1;
    bool alias_ = false;
    Tensor* placed_ = nullptr;          // a concat's tensor this copy writes into (not owned)
    long place_offset_ = 0, rows_per_block_ = 0, block_stride_ = 0;
};
REGISTER_KERNEL_WITH_NAME(ReshapeKernel, "Reshape");

// ----------------------------------------------------------------- Flatten
// nn/kernels/flatten.cc:16-96. Elements keep the stored (NHWC) order. For an
// NHWC4 input the ONNX axis is mapped onto the stored order as the reference does;
// where that leaves leading 1-sized dims (global-pool output [N,1,1,C], axis 1 ->
// 3) they are dropped so that the result is the 2-D [N, C] a following Gemm needs.
class FlattenKernel : public Kernel {
public:
    explicit FlattenKernel(Context* c) : Kernel(c) { kernel_fname_ = "reshape"; }
    void SetupAttr(const dlxnet::Attribute& attr) override { axis_ = attr.flatten_attr.axis; }
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK(IsPadded4(inputs[0]));
        nhwc_input_ = session_ && session_->IsONNX() && inputs[0]->dformat() == TP::NHWC4;
        output_tensor_dformats_.push_back(TP::ANY4);
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        const IntList& s = in[0];
        OGLE_CHECK(axis_ >= 0 && axis_ <= int(s.size()));
        out.assign(1, IntList());
        long tail = 1;
        if (nhwc_input_) {
            OGLE_CHECK_EQ(s.size(), 4u);
            // ONNX dims [N,C,H,W]: everything from `axis_` on is flattened; in stored order
            // that is a contiguous tail only for axis 1 (all of H,W,C) or axis 0
            OGLE_CHECK(axis_ <= 1) << "Flatten of an NHWC4 tensor supports axis 0 or 1";
            if (axis_ == 1) out[0].push_back(s[0]);
            for (size_t i = size_t(axis_); i < 4; ++i) tail *= s[i];
        } else {
            for (int i = 0; i < axis_; ++i) out[0].push_back(s[i]);
            for (size_t i = size_t(axis_); i < s.size(); ++i) tail *= s[i];
        }
        out[0].push_back(int(tail));
        n_ = 1;
        for (int d : s) n_ *= d;
        in_last_ = s.back();
        out_last_ = int(tail);
        alias_ = (in_last_ == out_last_) || (in_last_ % 4 == 0 && out_last_ % 4 == 0);
    }
    bool IsNoOp() const override { return alias_; }
    void Compute(TensorList& in, TensorList& out) override {
        if (alias_) return;
        OGLE_CUDA_OK(ogle_cuda_reshape(in[0]->device<float>(), out[0]->device<float>(), n_, in_last_, out_last_,
                                       context_->stream()));
    }
private:
    int axis_ = 1;
    bool nhwc_input_ = false, alias_ = false;
    long n_ = 0;
    int in_last_ = 1, out_last_ = 1;
};
REGISTER_KERNEL_WITH_NAME(FlattenKernel, "Flatten");

// ------------------------------------------------ Shape / Gather / Unsqueeze
// Shape arithmetic of exported graphs (Shape -> Gather -> Unsqueeze -> Concat ->
// Reshape). These only ever run in the setup pass; they go through the host.
class ShapeKernel : public Kernel {
public:
    explicit ShapeKernel(Context* c) : Kernel(c) { kernel_fname_ = "shape"; }
    void SetupAttr(const dlxnet::Attribute&) override {}
    bool ForceReady() const override { return true; }   // nn/kernels/shape.h
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        output_tensor_dformats_.push_back(TP::ANY4);
        OGLE_CHECK_EQ(in.size(), 1u);
        const int dims = int(in[0].size());
        out.assign(1, IntList{dims});
        tensor_.reset(new Tensor(Tensor::DT_FLOAT, IntList{dims}, Tensor::HOST_MEMORY, TP::ANY));
        for (int i = 0; i < dims; ++i) tensor_->host<float>()[i] = float(in[0][i]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        OGLE_CHECK_EQ(in.size(), 1u);
        context_->CopyCPUTensorToDevice(tensor_.get(), out[0]);
        context_->Synchronize();
    }
private:
    std::unique_ptr<Tensor> tensor_;
};
REGISTER_KERNEL_WITH_NAME(ShapeKernel, "Shape");

class GatherKernel : public Kernel {
public:
    explicit GatherKernel(Context* c) : Kernel(c) { kernel_fname_ = "gather"; }
    void SetupAttr(const dlxnet::Attribute& attr) override { axis_ = attr.gather_attr.axis; }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        output_tensor_dformats_.push_back(TP::ANY4);
        OGLE_CHECK_EQ(in.size(), 2u);
        out.assign(1, in[1]);
    }
    void Compute(TensorList& in, TensorList& out) override {
        // gather.glsl:7-18: a scalar index into a 4-element shape tensor, with the ONNX
        // (NCHW) index mapped onto the stored NHWC order: 0->0, 1->3, 2->1, 3->2
        Tensor data(Tensor::DT_FLOAT, in[0]->shape(), Tensor::HOST_MEMORY, TP::ANY);
        Tensor index(Tensor::DT_FLOAT, in[1]->shape(), Tensor::HOST_MEMORY, TP::ANY);
        context_->CopyDeviceTensorToCPU(in[0], &data);
        context_->CopyDeviceTensorToCPU(in[1], &index);
        OGLE_CHECK_GE(data.num_elements(), 1u);
        const int sel = int(index.host<float>()[0]);
        static const int lane[4] = {0, 3, 1, 2};
        const int src = lane[sel >= 0 && sel < 3 ? sel : 3];
        Tensor result(Tensor::DT_FLOAT, out[0]->shape(), Tensor::HOST_MEMORY, TP::ANY);
        std::memset(result.host(), 0, result.AllocatedSize());
        result.host<float>()[0] = size_t(src) < data.num_elements() ? data.host<float>()[src] : 0.f;
        context_->CopyCPUTensorToDevice(&result, out[0]);
        context_->Synchronize();
    }
private:
    int axis_ = 0;
};
REGISTER_KERNEL_WITH_NAME(GatherKernel, "Gather");

class UnsqueezeKernel : public Kernel {
public:
    explicit UnsqueezeKernel(Context* c) : Kernel(c) { kernel_fname_ = "unsqueeze"; }
    void SetupAttr(const dlxnet::Attribute& attr) override {
        for (int a : attr.unsqueeze_attr.axes) axes_.push_back(a);
        OGLE_CHECK_EQ(axes_.size(), 1u);   // unsqueeze.cc:22-24
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        output_tensor_dformats_.push_back(TP::ANY4);
        OGLE_CHECK_EQ(in.size(), 1u);
        out.assign(1, in[0]);
        OGLE_CHECK(axes_[0] >= 0 && axes_[0] <= int(in[0].size()));
        out[0].insert(out[0].begin() + axes_[0], 1);
        // inserting anywhere but after the last dim keeps the padded rows as they are
        alias_ = axes_[0] < int(in[0].size()) || in[0].empty();
        OGLE_CHECK(alias_) << "Unsqueeze: appending a trailing dim is not supported (unsqueeze.cc:55)";
    }
    bool IsNoOp() const override { return alias_; }
    void Compute(TensorList&, TensorList&) override {}
private:
    IntList axes_;
    bool alias_ = true;
};
REGISTER_KERNEL_WITH_NAME(UnsqueezeKernel, "Unsqueeze");

// ----------------------------------------------------------------- Decoder
// nn/kernels/decoder.cc:12-97: prediction [N,A,4] ANY4, anchors [N,h,w,4].
class DecoderKernel : public Kernel {
public:
    explicit DecoderKernel(Context* c) : Kernel(c) { kernel_fname_ = "ssd_decode"; }
    void SetupAttr(const dlxnet::Attribute&) override {}
    void SelectKernel(const TensorList& inputs) override {
        OGLE_CHECK_EQ(inputs.size(), 2u);
        OGLE_CHECK_EQ(inputs[0]->dformat(), TP::ANY4);
        output_tensor_dformats_.push_back(TP::ANY4);
    }
    void InferOutputShape(TensorShapeList& in, TensorShapeList& out) override {
        OGLE_CHECK_GE(in.size(), 2u);
        OGLE_CHECK_EQ(in[0].size(), 3u);
        OGLE_CHECK_EQ(in[0][2], 4);
        OGLE_CHECK_EQ(in[1].size(), 4u);
        OGLE_CHECK_EQ(in[1][0], in[0][0]);
        OGLE_CHECK_EQ(in[1][1] * in[1][2], in[0][1]);
        OGLE_CHECK_EQ(in[1][3], 4);
        // the reference reads anchors at the prediction's own index, i.e. one image
        OGLE_CHECK_EQ(in[0][0], 1) << "Decoder kernel is defined for batch 1; use functor::SSDBBoxDecoder for batches";
        out.assign(1, IntList{in[0][0], in[0][1], 4});
    }
    void Compute(TensorList& in, TensorList& out) override {
        const float var[4] = {0.1f, 0.1f, 0.2f, 0.2f};   // decoder.cc:18
        OGLE_CUDA_OK(ogle_cuda_ssd_decode(in[0]->device<float>(), in[1]->device<float>(), out[0]->device<float>(),
                                          in[0]->shape()[0], in[0]->shape()[1], var, context_->stream()));
    }
};
REGISTER_KERNEL_WITH_NAME(DecoderKernel, "Decoder");

}  // namespace
}  // namespace ogle

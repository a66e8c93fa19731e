#include "nn_ops.h"

#include <cstdlib>

#include "types.h"

namespace ogle {
namespace {

// One node, one output tensor, both called `name` (nn_ops.cc names them alike throughout).
dlxnet::NodeProto* NewNode(Scope* scope, const std::string& name, const char* type, const std::vector<int>& input_ids,
                           int* tensor_id) {
    dlxnet::NodeProto* node = scope->AddNode();
    node->name = name;
    node->type = type;
    for (int id : input_ids) node->input_index.push_back(id);
    *tensor_id = scope->AddTensor(name);
    node->output_index.push_back(*tensor_id);
    return node;
}

}  // namespace

int AddConstNode(Scope* scope, const std::string& name, const Tensor* cpu_tensor) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Const", {}, &id);
    cpu_tensor->AsProto(&node->attr.const_attr.value);
    return id;
}

int AddConstNode(Scope* scope, const std::string& name, const std::vector<int>& shape, DataFormat dst_dformat,
                 DataFormat src_dformat) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Const", {}, &id);
    dlxnet::TensorProto& t = node->attr.const_attr.value;
    size_t n = 1;
    for (int d : shape) {
        t.dims.push_back(d);
        n *= size_t(d);
    }
    t.float_data.resize(n);
    for (size_t j = 0; j < n; ++j) t.float_data[j] = float(1.0 * random() / RAND_MAX);
    t.data_type = dlxnet::TensorProto::FLOAT32;
    t.target_data_format = dst_dformat;
    t.data_format = src_dformat;
    return id;
}

int AddConvNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const Conv2dParams& p) {
    OGLE_CHECK_GT(p.dilation, 0);
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Conv", input_ids, &id);
    dlxnet::Conv2dAttribute& a = node->attr.conv2d_attr;
    a.kernel_shape.assign(2, p.kernel_size);
    a.strides.assign(2, p.stride);
    a.pads.assign(4, p.padding);
    a.group = p.groups;
    a.dilations.push_back(p.dilation);
    a.activation_type = p.activation_type;
    a.min = p.min;
    a.max = p.max;
    return id;
}

int AddInputNode(Scope* scope, std::string name) {
    scope->AddInputName(name);
    return scope->AddTensor(name);
}

int AddShapeNode(Scope* scope, std::string name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "Shape", input_ids, &id);
    return id;
}

int AddConcatNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const ConcatParams& p) {
    int id;
    NewNode(scope, name, "Concat", input_ids, &id)->attr.concat_attr.axis = p.axis;
    return id;
}

int AddReshapeNode(Scope* scope, const std::string& name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "Reshape", input_ids, &id);
    return id;
}

int AddTransposeNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const TransposeParams& p) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Transpose", input_ids, &id);
    for (int q : p.perm) node->attr.transpose_attr.perm.push_back(q);
    return id;
}

int AddClipNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const ClipParams& p) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Clip", input_ids, &id);
    node->attr.clip_attr.min = p.min;
    node->attr.clip_attr.max = p.max;
    return id;
}

int AddFlattenNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const FlattenParams& p) {
    int id;
    NewNode(scope, name, "Flatten", input_ids, &id)->attr.flatten_attr.axis = p.axis;
    return id;
}

int AddGemmNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const GemmParams& p) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "Gemm", input_ids, &id);
    node->attr.gemm_attr.alpha = p.alpha;
    node->attr.gemm_attr.beta = p.beta;
    node->attr.gemm_attr.transb = p.transb;
    return id;
}

int AddMaxPoolNode(Scope* scope, const std::string& name, std::vector<int> input_ids, const PoolParams& p) {
    int id;
    dlxnet::NodeProto* node = NewNode(scope, name, "MaxPool", input_ids, &id);
    node->attr.maxpool_attr.kernel_shape.assign(2, p.kernel_size);
    node->attr.maxpool_attr.strides.assign(2, p.stride);
    node->attr.maxpool_attr.pads.assign(4, p.padding);
    return id;
}

int AddGlobalAveragePoolNode(Scope* scope, const std::string& name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "GlobalAveragePool", input_ids, &id);
    return id;
}

int AddBatchNormNode(Scope* scope, const std::string& name, std::vector<int> input_ids, float epsilon) {
    int id;
    NewNode(scope, name, "BatchNormalization", input_ids, &id)->attr.batchnorm_attr.epsilon = epsilon;
    return id;
}

int AddReluNode(Scope* scope, const std::string& name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "Relu", input_ids, &id);
    return id;
}

int AddAddNode(Scope* scope, const std::string& name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "Add", input_ids, &id)->attr.binary_attr.binary_op_type = "Add";
    return id;
}

int AddDecoderNode(Scope* scope, const std::string& name, std::vector<int> input_ids) {
    int id;
    NewNode(scope, name, "Decoder", input_ids, &id);
    return id;
}

}  // namespace ogle

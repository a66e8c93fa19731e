#include "kernel.h"

#include "fbo_session.h"

namespace ogle {

void Kernel::Setup(const dlxnet::NodeProto& node, FBOSession* session) {
    // kernel.cc:29-46
    set_kernel_name(node.name);
    set_kernel_type(node.type);
    set_session(session);
    for (int64_t i : node.input_index) input_tensor_indexes_.push_back(int(i));
    for (int64_t i : node.output_index) output_tensor_indexes_.push_back(int(i));
    SetupAttr(node.attr);
}

DataFormat Kernel::GetOutputDFormat(int i) const {
    OGLE_CHECK_LT(i, int(output_tensor_dformats_.size())) << "in kernel " << kernel_name_ << " (" << kernel_type_ << ")";
    OGLE_CHECK_GE(i, 0);
    return output_tensor_dformats_[i];
}

void Kernel::InferOutputShape(const TensorList& inputs, TensorShapeList& output_shapes) {
    TensorShapeList input_shapes;
    for (auto t : inputs) input_shapes.push_back(t->shape());
    InferOutputShape(input_shapes, output_shapes);
}

std::string Kernel::DebugString() const {
    std::ostringstream ss;
    ss << "In kernel \n type: " << kernel_type() << " name: " << kernel_name() << "\n";
    auto dump = [&](const std::vector<int>& idx) {
        for (int id : idx) {
            Tensor* t = session_ ? session_->FindTensorById(id) : nullptr;
            ss << "(";
            if (t) for (int d : t->shape()) ss << d << " ";
            ss << ")[" << id << "], ";
        }
    };
    dump(input_tensor_indexes_);
    ss << "->";
    dump(output_tensor_indexes_);
    return ss.str();
}

}  // namespace ogle

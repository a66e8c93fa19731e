#include "scope.h"

namespace ogle {

Scope::Scope() {
    model_.producer_name = "ONNX";
    model_.version = "0.1";
    model_.doc_string = "ignored";
}

dlxnet::NodeProto* Scope::AddNode() {
    model_.graph.node.emplace_back();
    return &model_.graph.node.back();
}

void Scope::AddInputName(const std::string& name) { model_.graph.input_names.push_back(name); }

void Scope::AddOutputName(const std::string& name) { model_.graph.output_names.push_back(name); }

int Scope::AddTensor(const std::string& tensor_name) {
    model_.graph.tensor_names.push_back(tensor_name);
    return tensor_index_++;
}

}  // namespace ogle

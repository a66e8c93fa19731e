// In-memory graph builder: the runtime's twin of the reference's Scope
// (ogl_runtime/opengl/core/scope.h:9-35, scope.cc:5-33). Tests and tools build
// small graphs with it and hand ExportModel() to FBOSession::LoadGraph.
#ifndef OGLE_RUNTIME_SCOPE_H_
#define OGLE_RUNTIME_SCOPE_H_
#include <string>

#include "dlx.h"

namespace ogle {

class Scope {
public:
    // producer "ONNX", version "0.1" (scope.cc:5-11): sessions treat the graph as converter output
    Scope();
    // Appends an empty node to the graph and returns it for the caller to fill.
    // The pointer is valid until the next AddNode.
    dlxnet::NodeProto* AddNode();
    void AddInputName(const std::string& name);
    void AddOutputName(const std::string& name);
    // Registers a tensor name and returns its index (indices count up from 0).
    int AddTensor(const std::string& tensor_name);
    dlxnet::ModelProto ExportModel() const { return model_; }
    const dlxnet::GraphProto& graph() const { return model_.graph; }

private:
    int tensor_index_ = 0;
    dlxnet::ModelProto model_;
};

}  // namespace ogle
#endif

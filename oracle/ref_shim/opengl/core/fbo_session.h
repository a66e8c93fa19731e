// Test infrastructure only: a session that loads and runs nothing, so that the reference's
// Detector (examples/ssd/detector.cc) can be constructed on the CPU. The oracle fills the
// detector's host-side output tensors itself and drives only the post-process.
#ifndef ORACLE_REF_SHIM_OPENGL_CORE_FBO_SESSION_H_
#define ORACLE_REF_SHIM_OPENGL_CORE_FBO_SESSION_H_
#include "opengl/core/tensor.h"
#include "opengl/core/types.h"
namespace opengl {
class FBOSession {
public:
    void LoadGraph(const std::string&) {}
    bool allow_resized() const { return false; }
    const IntList& default_input_sizes() const { return sizes_; }
    void Run(const NamedTensorList&) { std::abort(); }
    Tensor* FindTensorByName(const std::string&) { std::abort(); }
    Context* context() { return &context_; }
private:
    IntList sizes_ = {1, 1};
    Context context_;
};
}  // namespace opengl
#endif

// Test infrastructure only: a host-memory stand-in for the reference's Tensor
// (ogl_runtime/opengl/core/tensor.h:72-280) carrying exactly the accessors that
// ogl_runtime/opengl/core/cpu_functor.cc calls, so that file compiles unmodified
// without the OpenGL headers the real tensor.h pulls in. The buffer is borrowed.
#ifndef ORACLE_REF_SHIM_OPENGL_CORE_TENSOR_H_
#define ORACLE_REF_SHIM_OPENGL_CORE_TENSOR_H_
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>
#include <glog/logging.h>
#define UP_DIV(x, y)   (((x) + (y) - (1)) / (y))
#define UP_ROUND(x, y) (((x) + (y) - (1)) / (y) * (y))
namespace opengl {
class Context {};
class Tensor {
public:
    Tensor(float* data, const std::vector<int>& shape, size_t allocated_elements)
        : data_(data), shape_(shape), allocated_(allocated_elements) {}
    bool is_host() const { return true; }
    template <typename T> T* host() const { return reinterpret_cast<T*>(data_); }
    const std::vector<int>& shape() const { return shape_; }
    size_t num_elements() const { size_t n = 1; for (int d : shape_) n *= size_t(d); return n; }
    int last_stride() const { return shape_.empty() ? 1 : shape_.back(); }
    uint64_t AllocatedSize() const { return allocated_ * sizeof(float); }
    uint64_t AllocatedElements() const { return allocated_; }
private:
    float* data_;
    std::vector<int> shape_;
    size_t allocated_;
};
}  // namespace opengl
#endif

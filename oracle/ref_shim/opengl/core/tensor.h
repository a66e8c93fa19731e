// Test infrastructure only: a host-memory stand-in for the reference's Tensor
// (ogl_runtime/opengl/core/tensor.h:72-280) carrying exactly the accessors that
// ogl_runtime/opengl/core/cpu_functor.cc and examples/ssd/detector.cc call, so that those
// files compile unmodified without the OpenGL headers the real tensor.h pulls in. The
// buffer is borrowed, except for tensors made by Empty() or the allocating constructor.
#ifndef ORACLE_REF_SHIM_OPENGL_CORE_TENSOR_H_
#define ORACLE_REF_SHIM_OPENGL_CORE_TENSOR_H_
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>
#include <glog/logging.h>
#include "opengl/core/types.h"
#define UP_DIV(x, y)   (((x) + (y) - (1)) / (y))
#define UP_ROUND(x, y) (((x) + (y) - (1)) / (y) * (y))
namespace opengl {
class Context {
public:
    void CopyDeviceTensorToCPU(const Tensor*, Tensor*) { std::abort(); }
};
class Tensor {
public:
    enum DataType { DT_INT = 0, DT_FLOAT = 1, DT_DOUBLE = 2, DT_INVALID };
    enum MemoryType { HOST_MEMORY = 0, DEVICE_TEXTURE, DEVICE_BUFFER };
    Tensor(float* data, const std::vector<int>& shape, size_t allocated_elements)
        : data_(data), shape_(shape), allocated_(allocated_elements) {}
    Tensor(DataType, const std::vector<int>& shape, MemoryType = HOST_MEMORY, DataFormat = dlxnet::TensorProto::NHWC)
        : shape_(shape), owned_(true) {
        allocated_ = num_elements();
        data_ = new float[allocated_ ? allocated_ : 1]();
    }
    static Tensor* Empty(DataType t, const std::vector<int>& shape, DataFormat f = dlxnet::TensorProto::NHWC) {
        return new Tensor(t, shape, HOST_MEMORY, f);
    }
    ~Tensor() { if (owned_) delete[] data_; }
    Tensor(const Tensor&) = delete;
    void operator=(const Tensor&) = delete;
    void* host() const { return data_; }
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
    bool owned_ = false;
};
}  // namespace opengl
#endif

// Tensor: shape + data format + one buffer, host or device.
// Mirrors ogl_runtime/opengl/core/tensor.h:72-280. Device tensors are linear
// CUDA buffers instead of RGBA32F textures:
//   NHWC4 / ANY4 : [prod(shape[:-1])][round_up(shape[-1],4)] floats - the byte
//                  layout of the reference's textures for those formats
//                  (tensor_format.cc:308-337);
//   HWN4C4       : a filter, kept dense in its OIHW order; the kernel that
//                  consumes it builds its own packed copy once, where the
//                  reference re-laid it out on upload (context.cc:143-145).
#ifndef OGLE_RUNTIME_TENSOR_H_
#define OGLE_RUNTIME_TENSOR_H_
#include "types.h"

namespace ogle {

inline int UpRound4(int v) { return (v + 3) / 4 * 4; }

bool IsStrideDFormat(DataFormat f);          // NHWC4, ANY4, HWN4C4
DataFormat FormatToStride4(DataFormat f);    // tensor_format.cc:171-187
DataFormat StrToFormat(const std::string& s);  // tensor_format.cc:136-152
// number of floats a tensor of this shape/format occupies (host or device)
uint64_t CalcAllocatedSize1D(const IntList& shape, DataFormat dformat);

class Tensor {
public:
    enum DataType { DT_INT = 0, DT_FLOAT = 1, DT_DOUBLE = 2, DT_INVALID };
    enum MemoryType { HOST_MEMORY = 0, DEVICE_TEXTURE, DEVICE_BUFFER };

    // Allocates; device tensors are allocated on the current CUDA device
    // (DEVICE_TEXTURE is kept as the name of "device memory").
    Tensor(DataType dtype, IntList shape, MemoryType mem_type = HOST_MEMORY,
           DataFormat dformat = dlxnet::TensorProto::NHWC);
    // Host tensor over caller-owned data (not freed).
    Tensor(DataType dtype, IntList shape, float* data, DataFormat dformat = dlxnet::TensorProto::NHWC);
    // Host tensor from a model constant; int tensors are stored as floats
    // (tensor.cc:69-81 writes int32 data through a float pointer).
    explicit Tensor(const dlxnet::TensorProto& proto);
    // Device tensor viewing memory owned elsewhere (an arena slot).
    Tensor(IntList shape, DataFormat dformat, float* device_ptr);
    ~Tensor();
    Tensor(const Tensor&) = delete;
    void operator=(const Tensor&) = delete;

    static Tensor* Random(DataType dtype, IntList shape, DataFormat dformat = dlxnet::TensorProto::NHWC);
    static Tensor* Empty(DataType dtype, IntList shape, DataFormat dformat = dlxnet::TensorProto::NHWC);
    static Tensor* Ones(DataType dtype, IntList shape, DataFormat dformat = dlxnet::TensorProto::NHWC);
    static Tensor* Zeros(DataType dtype, IntList shape, DataFormat dformat = dlxnet::TensorProto::NHWC);

    void* device() const { return device_; }
    void* host() const { return host_; }
    template <typename T> T* device() const { return reinterpret_cast<T*>(device_); }
    template <typename T> T* host() const { return reinterpret_cast<T*>(host_); }

    const IntList& shape() const { return shape_; }
    size_t num_elements() const { size_t n = 1; for (int d : shape_) n *= size_t(d); return n; }
    DataType dtype() const { return dtype_; }
    MemoryType mem_type() const { return mem_type_; }
    int dims_size() const { return int(shape_.size()); }
    DataFormat dformat() const { return dformat_; }
    void set_dformat(DataFormat f) { dformat_ = f; }
    bool is_host() const { return host_ != nullptr; }
    int last_stride() const { return shape_.empty() ? 1 : shape_.back(); }
    // floats per row of the device layout
    int padded_last() const { return IsStrideDFormat(dformat_) && dformat_ != dlxnet::TensorProto::HWN4C4 ? UpRound4(last_stride()) : last_stride(); }
    uint64_t AllocatedSize() const { return allocated_size_; }
    uint64_t AllocatedElements() const { return allocated_size_ / sizeof(float); }
    uint64_t RequestedSize() const { return num_elements() * sizeof(float); }
    void AsProto(dlxnet::TensorProto* proto) const;   // tensor.cc:167-186
    std::string ShortDebugString() const;

private:
    void* device_ = nullptr;
    void* host_ = nullptr;
    bool owns_ = true;
    uint64_t allocated_size_ = 0;
    DataType dtype_;
    MemoryType mem_type_;
    IntList shape_;
    DataFormat dformat_;
};

}  // namespace ogle
#endif

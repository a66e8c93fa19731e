#include "tensor.h"

#include <cuda_runtime.h>
#include <cstdlib>
#include <cstring>

namespace ogle {

bool IsStrideDFormat(DataFormat f) {
    return !(f == dlxnet::TensorProto::NHWC || f == dlxnet::TensorProto::NCHW || f == dlxnet::TensorProto::ANY);
}

DataFormat FormatToStride4(DataFormat f) {
    using T = dlxnet::TensorProto;
    if (f == T::NHWC || f == T::NHWC4) return T::NHWC4;
    if (f == T::ANY || f == T::ANY4) return T::ANY4;
    if (f == T::NCHW || f == T::HWN4C4) return T::HWN4C4;
    OGLE_FATAL() << "unsupported dformat: " << int(f);
}

DataFormat StrToFormat(const std::string& s) {
    using T = dlxnet::TensorProto;
    if (s == "NHWC") return T::NHWC;
    if (s == "NCHW") return T::NCHW;
    if (s == "ANY") return T::ANY;
    if (s == "NHWC4") return T::NHWC4;
    if (s == "ANY4") return T::ANY4;
    if (s == "HWN4C4") return T::HWN4C4;
    OGLE_FATAL() << "unsupported dformat_str: " << s;
}

uint64_t CalcAllocatedSize1D(const IntList& shape, DataFormat dformat) {
    using T = dlxnet::TensorProto;
    uint64_t n = 1;
    for (int d : shape) n *= uint64_t(d);
    const int last = shape.empty() ? 1 : shape.back();
    if (dformat == T::NHWC4 || dformat == T::ANY4) {
        if (last == 0) return 0;
        return n / uint64_t(last) * uint64_t(UpRound4(last));
    }
    // dense formats are rounded up to whole texels, as the reference does
    return (n + 3) / 4 * 4;
}

Tensor::Tensor(DataType dtype, IntList shape, MemoryType mem_type, DataFormat dformat)
    : dtype_(dtype), mem_type_(mem_type), shape_(std::move(shape)), dformat_(dformat) {
    if (shape_.size() != 4) {
        // tensor.h:239-245: non-4-D tensors are "general" tensors
        OGLE_CHECK(dformat_ == dlxnet::TensorProto::ANY || dformat_ == dlxnet::TensorProto::ANY4)
            << "a " << shape_.size() << "-D tensor must be ANY or ANY4";
    }
    allocated_size_ = CalcAllocatedSize1D(shape_, dformat_) * sizeof(float);
    const size_t bytes = allocated_size_ ? allocated_size_ : 16;
    if (mem_type_ == HOST_MEMORY) {
        host_ = std::malloc(bytes);
        OGLE_CHECK(host_ != nullptr) << "host allocation of " << bytes << " bytes failed";
    } else {
        cudaError_t e = cudaMalloc(&device_, bytes);
        OGLE_CHECK(e == cudaSuccess) << "cudaMalloc(" << bytes << "): " << cudaGetErrorString(e);
    }
}

Tensor::Tensor(DataType dtype, IntList shape, float* data, DataFormat dformat)
    : host_(data), owns_(false), dtype_(dtype), mem_type_(HOST_MEMORY), shape_(std::move(shape)), dformat_(dformat) {
    allocated_size_ = CalcAllocatedSize1D(shape_, dformat_) * sizeof(float);
}

Tensor::Tensor(IntList shape, DataFormat dformat, float* device_ptr)
    : device_(device_ptr), owns_(false), dtype_(DT_FLOAT), mem_type_(DEVICE_TEXTURE), shape_(std::move(shape)),
      dformat_(dformat) {
    allocated_size_ = CalcAllocatedSize1D(shape_, dformat_) * sizeof(float);
}

Tensor::Tensor(const dlxnet::TensorProto& p)
    : dtype_(DT_FLOAT), mem_type_(HOST_MEMORY), dformat_(p.data_format) {
    for (int d : p.dims) shape_.push_back(d);
    allocated_size_ = CalcAllocatedSize1D(shape_, dformat_) * sizeof(float);
    const size_t bytes = allocated_size_ ? allocated_size_ : 16;
    host_ = std::calloc(1, bytes);
    OGLE_CHECK(host_ != nullptr);
    float* dst = static_cast<float*>(host_);
    const size_t cap = allocated_size_ / sizeof(float);
    switch (p.data_type) {
        case dlxnet::TensorProto::FLOAT32:
            OGLE_CHECK_LE(p.float_data.size(), cap);
            std::memcpy(dst, p.float_data.data(), p.float_data.size() * sizeof(float));
            break;
        case dlxnet::TensorProto::INT32:
            dtype_ = DT_INT;
            OGLE_CHECK_LE(p.int32_data.size(), cap);
            for (size_t i = 0; i < p.int32_data.size(); ++i) dst[i] = float(p.int32_data[i]);
            break;
        default:
            OGLE_FATAL() << "unsupported const type: " << int(p.data_type);
    }
}

Tensor::~Tensor() {
    if (!owns_) return;
    if (host_) std::free(host_);
    if (device_) cudaFree(device_);
}

Tensor* Tensor::Empty(DataType dtype, IntList shape, DataFormat dformat) {
    return new Tensor(dtype, std::move(shape), HOST_MEMORY, dformat);
}
Tensor* Tensor::Zeros(DataType dtype, IntList shape, DataFormat dformat) {
    Tensor* t = Empty(dtype, std::move(shape), dformat);
    std::memset(t->host(), 0, t->AllocatedSize());
    return t;
}
Tensor* Tensor::Ones(DataType dtype, IntList shape, DataFormat dformat) {
    Tensor* t = Zeros(dtype, std::move(shape), dformat);
    const size_t n = t->num_elements();
    OGLE_CHECK(!IsStrideDFormat(dformat)) << "Ones/Random fill dense host formats";
    for (size_t i = 0; i < n; ++i) t->host<float>()[i] = 1.f;
    return t;
}
Tensor* Tensor::Random(DataType dtype, IntList shape, DataFormat dformat) {
    // uniform [0,1) from random(), as tensor.cc:104-115
    Tensor* t = Zeros(dtype, std::move(shape), dformat);
    OGLE_CHECK(!IsStrideDFormat(dformat)) << "Ones/Random fill dense host formats";
    const size_t n = t->num_elements();
    for (size_t i = 0; i < n; ++i) t->host<float>()[i] = float(1.0 * random() / RAND_MAX);
    return t;
}

void Tensor::AsProto(dlxnet::TensorProto* proto) const {
    OGLE_CHECK(is_host()) << "AsProto only used on host tensors";
    proto->dims.assign(shape_.begin(), shape_.end());
    proto->data_type = dlxnet::TensorProto::FLOAT32;
    proto->target_data_format = FormatToStride4(dformat_);
    proto->data_format = dformat_;
    const float* d = host<float>();
    proto->float_data.assign(d, d + num_elements());
}

std::string Tensor::ShortDebugString() const {
    std::ostringstream ss;
    ss << "Tensor(";
    for (size_t i = 0; i < shape_.size(); ++i) ss << (i ? "," : "") << shape_[i];
    ss << " fmt=" << int(dformat_) << (is_host() ? " host" : " device") << ")";
    return ss.str();
}

}  // namespace ogle

#include "context.h"

#include <cuda_runtime.h>
#include <cstdlib>

namespace ogle {

#define OGLE_RT_CUDA(call)                                                                   \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) OGLE_FATAL() << #call << ": " << cudaGetErrorString(e_);      \
    } while (0)

Context::Context(int device, ogle_stream_t stream) : device_(device), stream_(stream), owns_stream_(false) {
    if (device_ < 0) OGLE_RT_CUDA(cudaGetDevice(&device_));
    OGLE_RT_CUDA(cudaSetDevice(device_));
    if (!stream_) {
        cudaStream_t s;
        OGLE_RT_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        stream_ = reinterpret_cast<ogle_stream_t>(s);
        owns_stream_ = true;
    }
    if (const char* m = std::getenv("OGLE_MATH_MODE")) {
        const int v = std::atoi(m);
        if (v >= OGLE_MATH_FP32 && v <= OGLE_MATH_TF32X3) math_mode_ = v;
    }
}

Context::~Context() {
    cudaSetDevice(device_);
    if (staging_) cudaFree(staging_);
    if (owns_stream_) cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream_));
}

void Context::MakeCurrent() const { OGLE_RT_CUDA(cudaSetDevice(device_)); }
void Context::Synchronize() const { OGLE_RT_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream_))); }

float* Context::Staging(size_t bytes) {
    if (bytes > staging_bytes_) {
        // the old buffer may still be read by queued work
        Synchronize();
        if (staging_) OGLE_RT_CUDA(cudaFree(staging_));
        staging_ = nullptr;
        OGLE_RT_CUDA(cudaMalloc(&staging_, bytes));
        staging_bytes_ = bytes;
    }
    return staging_;
}

static void check_same_shape(const Tensor* a, const Tensor* b) {
    OGLE_CHECK_EQ(a->shape().size(), b->shape().size());
    for (size_t i = 0; i < a->shape().size(); ++i) OGLE_CHECK_EQ(a->shape()[i], b->shape()[i]);
}

void Context::CopyCPUTensorToDevice(const Tensor* cpu, Tensor* dev) {
    using T = dlxnet::TensorProto;
    OGLE_CHECK(cpu->is_host());
    OGLE_CHECK(!dev->is_host());
    check_same_shape(cpu, dev);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    const size_t n = cpu->num_elements();
    if (n == 0) return;
    const int last = cpu->last_stride();
    const DataFormat df = dev->dformat(), cf = cpu->dformat();
    const bool dev_padded = (df == T::NHWC4 || df == T::ANY4);
    const bool cpu_padded = (cf == T::NHWC4 || cf == T::ANY4);
    if (df == T::HWN4C4) {
        OGLE_CHECK(cf == T::NCHW || cf == T::ANY || cf == T::HWN4C4) << "filter upload from dformat " << int(cf);
        OGLE_RT_CUDA(cudaMemcpyAsync(dev->device(), cpu->host(), n * sizeof(float), cudaMemcpyHostToDevice, s));
        return;
    }
    OGLE_CHECK(dev_padded) << "unsupported conversion to device dformat " << int(df);
    if (cpu_padded || last % 4 == 0) {
        // same bytes on both sides (context.cc:125-133)
        OGLE_RT_CUDA(cudaMemcpyAsync(dev->device(), cpu->host(), dev->AllocatedSize(), cudaMemcpyHostToDevice, s));
        return;
    }
    OGLE_CHECK(cf == T::NHWC || cf == T::ANY || cf == T::NCHW)
        << "unsupported conversion from cpu dformat " << int(cf) << " to device dformat " << int(df);
    float* stage = Staging(n * sizeof(float));
    OGLE_RT_CUDA(cudaMemcpyAsync(stage, cpu->host(), n * sizeof(float), cudaMemcpyHostToDevice, s));
    OGLE_CUDA_OK(ogle_cuda_pad4(stage, dev->device<float>(), long(n / last), last, 0, stream_));
}

void Context::CopyDeviceTensorToCPU(const Tensor* dev, Tensor* cpu) {
    using T = dlxnet::TensorProto;
    OGLE_CHECK(cpu->is_host());
    OGLE_CHECK(!dev->is_host());
    check_same_shape(cpu, dev);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
    const size_t n = cpu->num_elements();
    if (n == 0) return;
    const int last = cpu->last_stride();
    const DataFormat df = dev->dformat(), cf = cpu->dformat();
    const bool cpu_padded = (cf == T::NHWC4 || cf == T::ANY4);
    if (df == T::HWN4C4) {
        OGLE_CHECK(cf == T::NCHW || cf == T::ANY || cf == T::HWN4C4) << "filter readback to dformat " << int(cf);
        OGLE_RT_CUDA(cudaMemcpyAsync(cpu->host(), dev->device(), n * sizeof(float), cudaMemcpyDeviceToHost, s));
    } else if (cpu_padded || last % 4 == 0) {
        OGLE_RT_CUDA(cudaMemcpyAsync(cpu->host(), dev->device(), dev->AllocatedSize(), cudaMemcpyDeviceToHost, s));
    } else {
        OGLE_CHECK(cf == T::NHWC || cf == T::ANY) << "unsupported conversion from device dformat " << int(df)
                                                   << " -> cpu dformat " << int(cf);
        float* stage = Staging(n * sizeof(float));
        OGLE_CUDA_OK(ogle_cuda_unpad4(dev->device<float>(), stage, long(n / last), last, 0, stream_));
        OGLE_RT_CUDA(cudaMemcpyAsync(cpu->host(), stage, n * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    Synchronize();
}

Context* GetContext() {
    static Context* context = new Context;
    return context;
}

}  // namespace ogle

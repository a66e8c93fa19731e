// Context: the device side of a session - CUDA device, stream, and the
// host<->device copies with layout conversion. Takes the role of the
// reference's Context (ogl_runtime/opengl/core/context.h:15-86), whose GL
// program cache and framebuffer have no counterpart here: kernels are compiled
// ahead of time into libogle_cuda.so.
#ifndef OGLE_RUNTIME_CONTEXT_H_
#define OGLE_RUNTIME_CONTEXT_H_
#include "ogle_cuda.h"
#include "tensor.h"

namespace ogle {

class Context {
public:
    // device < 0: keep the calling thread's current device. stream == nullptr: create one.
    explicit Context(int device = -1, ogle_stream_t stream = nullptr);
    ~Context();

    int device() const { return device_; }
    ogle_stream_t stream() const { return stream_; }
    // The stream kernels enqueue on. A session swaps it while it records independent
    // branches of a graph on side streams, and puts the original back.
    void set_stream(ogle_stream_t s) { stream_ = s; }
    void MakeCurrent() const;
    void Synchronize() const;

    // context.cc:123-154 - upload with conversion: dense NHWC/ANY -> NHWC4/ANY4
    // (zero-padded channels), NCHW/ANY filter -> HWN4C4 (kept dense). Asynchronous on
    // stream(); the host buffer must stay valid until the stream reaches the copy.
    void CopyCPUTensorToDevice(const Tensor* cpu_tensor, Tensor* device_tensor);
    // context.cc:157-185 - readback with the inverse conversion. Synchronises the
    // stream before returning (glReadPixels is the reference's only implicit sync too).
    void CopyDeviceTensorToCPU(const Tensor* device_tensor, Tensor* cpu_tensor);

    // Default math mode for dense contractions created through this context.
    int math_mode() const { return math_mode_; }
    void set_math_mode(int m) { math_mode_ = m; }

    // Grow-only device scratch for the copy conversions (never shrinks; sized at
    // the first call, so steady-state runs do not allocate).
    float* Staging(size_t bytes);

private:
    int device_;
    ogle_stream_t stream_;
    bool owns_stream_;
    int math_mode_ = OGLE_MATH_TF32X3;
    float* staging_ = nullptr;
    size_t staging_bytes_ = 0;
};

// Process-wide default context on the current device (context.cc:316-319).
Context* GetContext();

}  // namespace ogle
#endif

// Device functors used outside the graph, as ogl_runtime/opengl/core/functor.h.
#ifndef OGLE_RUNTIME_FUNCTOR_H_
#define OGLE_RUNTIME_FUNCTOR_H_
#include "context.h"

namespace ogle {
namespace functor {

// functor.cc:96-143: prediction [N,A,4] (ANY4), anchors [A,4] (ANY4), decoded
// [N,A,4]; all on the device. Anchors are shared by every image of the batch
// (the reference defines N == 1 only).
struct SSDBBoxDecoder {
    void operator()(Context* ctx, const Tensor* prediction_tensor, const Tensor* anchor_tensor,
                    Tensor* decoded_tensor, const std::vector<float>& variances);
};

}  // namespace functor
}  // namespace ogle
#endif

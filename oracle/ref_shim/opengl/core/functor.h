// Test infrastructure only: the device box decoder is not part of what the oracle drives in
// the reference's detector; its CPU twin (core/cpu_functor.cc) is compiled separately.
#ifndef ORACLE_REF_SHIM_OPENGL_CORE_FUNCTOR_H_
#define ORACLE_REF_SHIM_OPENGL_CORE_FUNCTOR_H_
#include "opengl/core/tensor.h"
namespace opengl {
namespace functor {
struct SSDBBoxDecoder {
    void operator()(Context*, const Tensor*, const Tensor*, Tensor*, const std::vector<float>&) { std::abort(); }
};
}  // namespace functor
}  // namespace opengl
#endif

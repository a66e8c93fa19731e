// Test infrastructure only: the type aliases of the reference's core/types.h that its
// SSD example uses, without the generated protobuf header the real file includes.
#ifndef ORACLE_REF_SHIM_OPENGL_CORE_TYPES_H_
#define ORACLE_REF_SHIM_OPENGL_CORE_TYPES_H_
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>
namespace dlxnet {
struct TensorProto {
    enum DataFormat { NCHW = 0, NHWC = 1, ANY = 2, NHWC4 = 3, HWN4C4 = 4, ANY4 = 5 };
};
}  // namespace dlxnet
namespace opengl {
class Tensor;
class Context;
typedef std::vector<int> IntList;
typedef std::vector<Tensor*> TensorList;
typedef std::vector<std::string> StringList;
typedef std::vector<std::string> TensorNameList;
typedef std::vector<std::pair<std::string, Tensor*>> NamedTensorList;
typedef dlxnet::TensorProto::DataFormat DataFormat;
typedef std::string string;
}  // namespace opengl
#endif

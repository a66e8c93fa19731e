// String-keyed operator registry with static-initialisation registration, as
// ogl_runtime/opengl/core/kernel_registry.h:8-42. The key is the dlx node type,
// which is the ONNX operator name.
#ifndef OGLE_RUNTIME_KERNEL_REGISTRY_H_
#define OGLE_RUNTIME_KERNEL_REGISTRY_H_
#include "types.h"

namespace ogle {

class KernelRegistry {
public:
    void RegisterKernel(const std::string& kernel_name, KernelFactory kernel_factory);
    // Leaves *kernel untouched (null) for an unknown name; the session reports it.
    void CreateKernel(const std::string& kernel_name, Kernel** kernel, Context* context);
    std::vector<std::string> RegisteredNames() const;
    static KernelRegistry* Global();

private:
    KernelRegistry() {}
    mutable KernelMap kernel_map_;
};

namespace registry {
template <typename T>
class KernelRegisterHelper {
public:
    explicit KernelRegisterHelper(const char* kernel_name) {
        KernelRegistry::Global()->RegisterKernel(std::string(kernel_name),
                                                 [](Kernel** kernel, Context* context) { *kernel = new T(context); });
    }
};
}  // namespace registry
}  // namespace ogle

#define REGISTER_KERNEL_UNIQ(ctr, Class, class_name) \
    static auto __register##ctr = ::ogle::registry::KernelRegisterHelper<Class>(class_name)
#define REGISTER_KERNEL_UNIQ_HELPER(ctr, Class, name) REGISTER_KERNEL_UNIQ(ctr, Class, name)
#define REGISTER_KERNEL(Class) REGISTER_KERNEL_UNIQ_HELPER(__COUNTER__, Class, #Class)
#define REGISTER_KERNEL_WITH_NAME(Class, class_name) REGISTER_KERNEL_UNIQ_HELPER(__COUNTER__, Class, class_name)

#endif

#include "kernel_registry.h"

#include <algorithm>

namespace ogle {

KernelRegistry* KernelRegistry::Global() {
    static KernelRegistry* registry = new KernelRegistry;
    return registry;
}

void KernelRegistry::RegisterKernel(const std::string& kernel_name, KernelFactory kernel_factory) {
    kernel_map_[kernel_name] = kernel_factory;
}

void KernelRegistry::CreateKernel(const std::string& kernel_name, Kernel** kernel, Context* context) {
    auto it = kernel_map_.find(kernel_name);
    if (it == kernel_map_.end()) return;   // kernel_registry.cc:19-23
    it->second(kernel, context);
}

std::vector<std::string> KernelRegistry::RegisteredNames() const {
    std::vector<std::string> names;
    for (auto& kv : kernel_map_) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    return names;
}

}  // namespace ogle

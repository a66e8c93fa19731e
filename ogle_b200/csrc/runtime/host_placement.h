// Host-side placement for one-process-per-GPU (or one-thread-per-GPU) serving: the thread that
// feeds a GPU, and the pinned buffers it uploads from, belong on the NUMA node the GPU's PCIe
// root port hangs off. With eight GPUs on two sockets, buffers that all sit on one socket make
// every upload of the other four GPUs cross the inter-socket link and share one socket's DRAM.
// The reference runs one GL context on one thread (core/init.cc:21-43) and has no counterpart.
#ifndef OGLE_RUNTIME_HOST_PLACEMENT_H_
#define OGLE_RUNTIME_HOST_PLACEMENT_H_

#include <string>
#include <vector>

namespace ogle {

// "0-3,8,10-11" -> {0,1,2,3,8,10,11}. Malformed pieces are skipped.
std::vector<int> ParseCpuList(const std::string& text);

struct HostPlacement {
    int numa_node = -1;        // node of the device's PCI function; -1 = unknown / single node
    int cpus_bound = 0;        // CPUs in the calling thread's new affinity mask; 0 = affinity left alone
    bool memory_preferred = false;   // the calling thread's page allocations now prefer numa_node
    std::string pci_bus_id;
};

// Looks up the device's NUMA node (sysfs), narrows the calling thread's CPU affinity to that
// node's CPUs (only those it was already allowed to use; untouched if none are), and sets the
// thread's memory policy to prefer that node, so that host buffers allocated afterwards
// (pinned or not) are local to the GPU. Never fails: what cannot be done is reported in the result.
HostPlacement BindHostToDevice(int device);

// Pinned host memory for upload buffers: anonymous memory advised to use 2 MB pages
// (transparent huge pages, where the host grants them), touched, then registered with CUDA.
// Uploads from it need fewer IOMMU translations than from 4 KB pages. Whether the host
// granted 2 MB pages is reported by HugePageBytes. Returns nullptr when the mapping or the
// registration fails. Free with FreePinnedHost only.
void* AllocPinnedHost(size_t bytes);
void FreePinnedHost(void* p);
// Bytes of the mapping that holds `p` which the kernel backs with 2 MB pages right now
// (AnonHugePages + ShmemPmdMapped of its /proc/self/smaps entry); 0 when none or unknown.
size_t HugePageBytes(const void* p);

// A named region of host memory shared by the processes of one box (POSIX shared memory),
// for one-process-per-GPU serving of ONE batch: the process that owns the batch writes the
// images once, every process uploads its own images straight from the region, and every
// process's detections are copied from its GPU straight into the region, where the owner
// reads them - no copy between processes, no collective. `create` makes (or truncates) the
// object and zero-fills it, otherwise an existing one of at least `bytes` is mapped. With
// `pin` the mapping is registered with CUDA in the calling process (its device context must
// be current), which makes copies from and to it asynchronous. Returns nullptr on failure
// (the reason in *error when given). Close with CloseSharedHost; `unlink` removes the name
// (the creator does that once every process has opened it or at shutdown).
void* OpenSharedHost(const std::string& name, size_t bytes, bool create, bool pin, std::string* error = nullptr);
void CloseSharedHost(void* p, bool unlink);

}  // namespace ogle

#endif

#include "host_placement.h"

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <sys/mman.h>

#include <cctype>
#include <cstring>
#include <map>
#include <mutex>
#include <cstdlib>
#include <fstream>

namespace ogle {

std::vector<int> ParseCpuList(const std::string& text) {
    std::vector<int> cpus;
    size_t i = 0;
    const size_t n = text.size();
    auto number = [&](int* out) {
        if (i >= n || !std::isdigit(static_cast<unsigned char>(text[i]))) return false;
        long v = 0;
        while (i < n && std::isdigit(static_cast<unsigned char>(text[i]))) {
            v = v * 10 + (text[i] - '0');
            if (v > 1 << 20) return false;
            ++i;
        }
        *out = int(v);
        return true;
    };
    while (i < n) {
        int lo = 0, hi = 0;
        if (number(&lo)) {
            hi = lo;
            if (i < n && text[i] == '-') {
                ++i;
                if (!number(&hi)) hi = lo - 1;      // "3-" : skip
            }
            for (int c = lo; c <= hi; ++c) cpus.push_back(c);
        }
        while (i < n && text[i] != ',') ++i;        // skip to the next piece
        if (i < n) ++i;
    }
    return cpus;
}

namespace {

bool ReadLine(const std::string& path, std::string* out) {
    std::ifstream f(path);
    if (!f) return false;
    std::getline(f, *out);
    return true;
}

}  // namespace

HostPlacement BindHostToDevice(int device) {
    HostPlacement r;
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, int(sizeof(bus)), device) != cudaSuccess) {
        cudaGetLastError();
        return r;
    }
    for (char* p = bus; *p; ++p) *p = char(std::tolower(static_cast<unsigned char>(*p)));
    r.pci_bus_id = bus;
    const std::string dir = std::string("/sys/bus/pci/devices/") + bus;
    std::string line;
    if (!ReadLine(dir + "/numa_node", &line)) return r;
    r.numa_node = std::atoi(line.c_str());
    if (r.numa_node < 0) return r;

    // CPU affinity: the node's CPUs among those this thread may already use
    if (ReadLine(dir + "/local_cpulist", &line)) {
        cpu_set_t allowed, want;
        CPU_ZERO(&want);
        if (sched_getaffinity(0, sizeof(allowed), &allowed) == 0) {
            int count = 0;
            for (int c : ParseCpuList(line))
                if (c < CPU_SETSIZE && CPU_ISSET(c, &allowed)) { CPU_SET(c, &want); ++count; }
            if (count > 0 && sched_setaffinity(0, sizeof(want), &want) == 0) r.cpus_bound = count;
        }
    }
    // memory policy of this thread: prefer the node (falls back to others when it is full or
    // not allowed). MPOL_PREFERRED = 1 in the kernel's mempolicy interface.
    if (r.numa_node < 1024) {
        unsigned long mask[1024 / (8 * sizeof(unsigned long))] = {0};
        mask[r.numa_node / (8 * sizeof(unsigned long))] |= 1ul << (r.numa_node % (8 * sizeof(unsigned long)));
        if (syscall(SYS_set_mempolicy, 1, mask, 1024ul) == 0) r.memory_preferred = true;
    }
    return r;
}

namespace {
struct Mapping { void* base; size_t length; };
std::mutex g_pinned_mutex;
std::map<void*, Mapping> g_pinned;
}  // namespace

void* AllocPinnedHost(size_t bytes) {
    if (bytes == 0) return nullptr;
    const size_t huge = size_t(2) << 20;
    const size_t length = (bytes + huge - 1) / huge * huge + huge;      // room to align the start
    void* base = mmap(nullptr, length, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (base == MAP_FAILED) return nullptr;
#ifdef MADV_HUGEPAGE
    madvise(base, length, MADV_HUGEPAGE);                               // best effort
#endif
    char* p = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(base) + huge - 1) / huge * huge);
    std::memset(p, 0, bytes);                                           // the pages exist before they are pinned
    if (cudaHostRegister(p, bytes, cudaHostRegisterDefault) != cudaSuccess) {
        cudaGetLastError();
        munmap(base, length);
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_pinned_mutex);
    g_pinned[p] = Mapping{base, length};
    return p;
}

void FreePinnedHost(void* p) {
    if (!p) return;
    Mapping m{nullptr, 0};
    {
        std::lock_guard<std::mutex> lock(g_pinned_mutex);
        auto it = g_pinned.find(p);
        if (it == g_pinned.end()) return;
        m = it->second;
        g_pinned.erase(it);
    }
    cudaHostUnregister(p);
    munmap(m.base, m.length);
}

}  // namespace ogle

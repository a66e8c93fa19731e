#include "host_placement.h"

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>

#include <cerrno>
#include <sstream>

#include <cctype>
#include <cstdio>
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
struct Mapping { void* base; size_t length; bool pinned = true; std::string shared_name; };
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
    Mapping m;
    m.base = base; m.length = length;
    g_pinned[p] = m;
    return p;
}

size_t HugePageBytes(const void* p) {
    // /proc/self/smaps: a header line "lo-hi perms ..." per mapping, then "Key:   value kB" lines
    std::ifstream f("/proc/self/smaps");
    if (!f) return 0;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
    std::string line;
    bool inside = false;
    size_t kb = 0;
    while (std::getline(f, line)) {
        unsigned long lo = 0, hi = 0;
        if (std::sscanf(line.c_str(), "%lx-%lx ", &lo, &hi) == 2 && line.find(':') > line.find(' ')) {
            if (inside) break;
            inside = addr >= lo && addr < hi;
            continue;
        }
        if (!inside) continue;
        unsigned long v = 0;
        if (std::sscanf(line.c_str(), "AnonHugePages: %lu kB", &v) == 1) kb += v;
        else if (std::sscanf(line.c_str(), "ShmemPmdMapped: %lu kB", &v) == 1) kb += v;
    }
    return kb * 1024;
}

void* OpenSharedHost(const std::string& name, size_t bytes, bool create, bool pin, std::string* error) {
    auto fail = [&](const std::string& what) -> void* {
        if (error) *error = what + ": " + std::strerror(errno);
        return nullptr;
    };
    if (bytes == 0 || name.empty() || name[0] != '/') {
        if (error) *error = "shared region needs a name that starts with '/' and a size";
        return nullptr;
    }
    const int fd = create ? shm_open(name.c_str(), O_CREAT | O_RDWR | O_TRUNC, 0600) : shm_open(name.c_str(), O_RDWR, 0600);
    if (fd < 0) return fail("shm_open(" + name + ")");
    if (create) {
        if (ftruncate(fd, off_t(bytes)) != 0) { close(fd); return fail("ftruncate"); }
    } else {
        struct stat st;
        if (fstat(fd, &st) != 0 || size_t(st.st_size) < bytes) {
            close(fd);
            if (error) *error = "shared region " + name + " is smaller than the size asked for";
            return nullptr;
        }
    }
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return fail("mmap");
#ifdef MADV_HUGEPAGE
    madvise(p, bytes, MADV_HUGEPAGE);                                   // best effort (shmem huge pages)
#endif
    if (create) std::memset(p, 0, bytes);                               // the pages exist before they are pinned
    if (pin) {
        // every process touches its own page tables before the registration walks them
        volatile const char* q = static_cast<const char*>(p);
        char sink = 0;
        for (size_t i = 0; i < bytes; i += 4096) sink ^= q[i];
        (void)sink;
        const cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable);
        if (e != cudaSuccess) {
            cudaGetLastError();
            munmap(p, bytes);
            if (error) *error = std::string("cudaHostRegister: ") + cudaGetErrorString(e);
            return nullptr;
        }
    }
    std::lock_guard<std::mutex> lock(g_pinned_mutex);
    Mapping m;
    m.base = p; m.length = bytes; m.pinned = pin; m.shared_name = name;
    g_pinned[p] = m;
    return p;
}

void CloseSharedHost(void* p, bool unlink) {
    if (!p) return;
    Mapping m;
    {
        std::lock_guard<std::mutex> lock(g_pinned_mutex);
        auto it = g_pinned.find(p);
        if (it == g_pinned.end() || it->second.shared_name.empty()) return;
        m = it->second;
        g_pinned.erase(it);
    }
    if (m.pinned) cudaHostUnregister(p);
    munmap(m.base, m.length);
    if (unlink) shm_unlink(m.shared_name.c_str());
}

void FreePinnedHost(void* p) {
    if (!p) return;
    Mapping m;
    {
        std::lock_guard<std::mutex> lock(g_pinned_mutex);
        auto it = g_pinned.find(p);
        if (it == g_pinned.end() || !it->second.shared_name.empty()) return;
        m = it->second;
        g_pinned.erase(it);
    }
    cudaHostUnregister(p);
    munmap(m.base, m.length);
}

}  // namespace ogle

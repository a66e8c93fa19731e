// Common typedefs of the host runtime; same names as the reference's
// ogl_runtime/opengl/core/types.h:13-41.
#ifndef OGLE_RUNTIME_TYPES_H_
#define OGLE_RUNTIME_TYPES_H_
#include <cstdint>
#include <functional>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "dlx.h"

namespace ogle {

class Kernel;
class Context;
class Tensor;

typedef std::vector<int> IntList;
typedef std::vector<Tensor*> TensorList;
typedef std::vector<IntList> TensorShapeList;
typedef std::vector<std::unique_ptr<Kernel>> OwnedKernelList;
typedef std::vector<std::unique_ptr<Tensor>> OwnedTensorList;
typedef std::vector<std::string> StringList;
typedef std::function<void(Kernel**, Context*)> KernelFactory;
typedef std::unordered_map<std::string, KernelFactory> KernelMap;
typedef std::unordered_map<std::string, int> NamedIndex;
typedef std::vector<std::string> TensorNameList;
typedef std::vector<std::pair<std::string, Tensor*>> NamedTensorList;
typedef dlxnet::TensorProto::DataFormat DataFormat;

// The reference aborts the process on every failed CHECK / LOG(FATAL)
// (e.g. conv2d.cc:71-86, fbo_session.cc:112-115). A library must not abort its
// host, so the same conditions throw FatalError here; the C ABI turns it into
// an error status plus message.
class FatalError : public std::runtime_error {
public:
    explicit FatalError(const std::string& m) : std::runtime_error(m) {}
};

namespace detail {
class FatalStream {
public:
    FatalStream(const char* file, int line, const char* cond) {
        ss_ << file << ":" << line << " ";
        if (cond) ss_ << "Check failed: " << cond << " ";
    }
    template <class T> FatalStream& operator<<(const T& v) { ss_ << v; return *this; }
    [[noreturn]] void raise() const { throw FatalError(ss_.str()); }
private:
    std::ostringstream ss_;
};
struct Raiser { [[noreturn]] void operator&(const FatalStream& s) const { s.raise(); } };
}  // namespace detail

}  // namespace ogle

#define OGLE_FATAL() ::ogle::detail::Raiser() & ::ogle::detail::FatalStream(__FILE__, __LINE__, nullptr)
// `switch (0) case 0: default:` keeps a following `else` from pairing with this `if`
#define OGLE_CHECK(cond) \
    switch (0) case 0: default: if (cond) {} else ::ogle::detail::Raiser() & ::ogle::detail::FatalStream(__FILE__, __LINE__, #cond)
#define OGLE_CHECK_EQ(a, b) OGLE_CHECK((a) == (b)) << "(" << (a) << " vs " << (b) << ") "
#define OGLE_CHECK_GE(a, b) OGLE_CHECK((a) >= (b)) << "(" << (a) << " vs " << (b) << ") "
#define OGLE_CHECK_GT(a, b) OGLE_CHECK((a) > (b)) << "(" << (a) << " vs " << (b) << ") "
#define OGLE_CHECK_LE(a, b) OGLE_CHECK((a) <= (b)) << "(" << (a) << " vs " << (b) << ") "
#define OGLE_CHECK_LT(a, b) OGLE_CHECK((a) < (b)) << "(" << (a) << " vs " << (b) << ") "
// status of a C-ABI call into libogle_cuda
#define OGLE_CUDA_OK(call)                                                              \
    do {                                                                                \
        const int ogle_rc_ = (call);                                                    \
        if (ogle_rc_ != 0)                                                              \
            OGLE_FATAL() << #call << " -> " << ogle_cuda_status_string(ogle_rc_) << " " \
                         << ogle_cuda_last_error();                                     \
    } while (0)

// Reference-style code can keep spelling the namespace `opengl`.
namespace opengl = ogle;

#endif

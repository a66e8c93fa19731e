// Test infrastructure only: the few glog macros the reference's CPU functors and its SSD
// example use, so that ogl_runtime/opengl/core/cpu_functor.cc and examples/ssd/*.cc
// compile without the glog library. A failed check aborts, as glog's does; LOG and VLOG
// messages are dropped.
#ifndef ORACLE_REF_SHIM_GLOG_LOGGING_H_
#define ORACLE_REF_SHIM_GLOG_LOGGING_H_
#include <cstdio>
#include <cstdlib>
#include <iostream>
namespace ref_shim {
struct Voidify { void operator&(std::ostream&) {} };
struct FatalStream {
    std::ostream& stream() { return std::cerr; }
    ~FatalStream() { std::cerr << std::endl; std::abort(); }
};
}  // namespace ref_shim
#define CHECK(cond) (cond) ? (void)0 : ref_shim::Voidify() & ref_shim::FatalStream().stream() << "Check failed: " #cond " "
#define CHECK_NOTNULL(p) CHECK((p) != nullptr)
#define LOG(severity) true ? (void)0 : ref_shim::Voidify() & std::cerr
#define VLOG(level) true ? (void)0 : ref_shim::Voidify() & std::cerr
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_NE(a, b) CHECK((a) != (b))
#define CHECK_GE(a, b) CHECK((a) >= (b))
#define CHECK_GT(a, b) CHECK((a) > (b))
#define CHECK_LE(a, b) CHECK((a) <= (b))
#define CHECK_LT(a, b) CHECK((a) < (b))
#endif

// Test infrastructure only: the few glog macros the reference's CPU functors
// use (CHECK, CHECK_EQ, CHECK_GE), so that ogl_runtime/opengl/core/cpu_functor.cc
// compiles without the glog library. A failed check aborts, as glog's does.
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
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_NE(a, b) CHECK((a) != (b))
#define CHECK_GE(a, b) CHECK((a) >= (b))
#define CHECK_GT(a, b) CHECK((a) > (b))
#define CHECK_LE(a, b) CHECK((a) <= (b))
#define CHECK_LT(a, b) CHECK((a) < (b))
#endif

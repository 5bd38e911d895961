/*
 * Stand-in for the reference project's include/raf/device.h, TEST INFRASTRUCTURE ONLY.
 *
 * The reference's CUDA kernel files (src/op/dialect/cuda/kernels/*.cu) include src/common/cuda_utils.h, which
 * includes "raf/device.h" for one type (raf::DType) used by helper templates the kernels never call.  The real header
 * pulls in TVM and dlpack, which are un-vendored submodules of the reference.  This file declares just enough for
 * cuda_utils.h to parse, so that the kernel files compile unmodified from where they lie; it defines no behaviour
 * of the kernels themselves.
 */
#pragma once
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <sstream>
#include <type_traits>

namespace raf_ref_stub {
struct Fatal {
  std::ostringstream os;
  template <typename T>
  Fatal& operator<<(const T& v) {
    os << v;
    return *this;
  }
  ~Fatal() {
    std::fprintf(stderr, "%s\n", os.str().c_str());
    std::abort();
  }
};
struct Voidify {
  void operator&(Fatal&) {}
};
}  // namespace raf_ref_stub

#define FATAL 0
#define LOG(severity) ::raf_ref_stub::Fatal()
#define CHECK(cond) (cond) ? (void)0 : ::raf_ref_stub::Voidify() & ::raf_ref_stub::Fatal() << "Check failed: " #cond " "

enum { kDLInt = 0, kDLUInt = 1, kDLFloat = 2 };

namespace raf {
class DType {
 public:
  int code{kDLFloat};
  int bits{32};
  int lanes{1};
  const char* c_str() const { return "dtype"; }
  template <typename T>
  operator T() const;
};
}  // namespace raf

// Stand-in for <glog/logging.h> (glog 0.7.x), written for the checker build only.
//
// TEST INFRASTRUCTURE.  The reference project's CPU kernels include glog, which is not
// installed where this checker is built.  Their sources use only LOG(severity) << ...,
// CHECK(cond) << ... and the CHECK_xx(a, b) comparisons; this header gives those the same
// observable behaviour (a message on stderr; FATAL and a failed CHECK abort) so that the
// reference's .cpp files compile unmodified.  Nothing in the product library includes it.
#pragma once
// glog's header pulls in a good part of the standard library, and the reference's sources
// lean on that (std::vector, std::memcpy, std::string without their own includes).
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <iostream>
#include <limits>
#include <memory>
#include <sstream>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace shim_glog {
enum Severity { INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };

class Message {
 public:
  Message(const char* file, int line, Severity sev) : sev_(sev) {
    static const char tag[] = {'I', 'W', 'E', 'F'};
    os_ << tag[sev] << ' ' << file << ':' << line << "] ";
  }
  ~Message() {
    if (sev_ >= WARNING) std::cerr << os_.str() << std::endl;
    if (sev_ == FATAL) std::abort();
  }
  std::ostream& stream() { return os_; }

 private:
  Severity sev_;
  std::ostringstream os_;
};

// Lets `cond ? (void)0 : Voidify() & stream` type-check: & binds looser than <<.
struct Voidify {
  void operator&(std::ostream&) {}
};
}  // namespace shim_glog

#define LOG(severity) ::shim_glog::Message(__FILE__, __LINE__, ::shim_glog::severity).stream()
#define CHECK(cond)                                                                      \
  (cond) ? (void)0                                                                       \
         : ::shim_glog::Voidify() &                                                      \
               ::shim_glog::Message(__FILE__, __LINE__, ::shim_glog::FATAL).stream()     \
                   << "Check failed: " #cond " "
#define SHIM_CHECK_OP(a, b, op) CHECK((a)op(b))
#define CHECK_EQ(a, b) SHIM_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) SHIM_CHECK_OP(a, b, !=)
#define CHECK_LT(a, b) SHIM_CHECK_OP(a, b, <)
#define CHECK_LE(a, b) SHIM_CHECK_OP(a, b, <=)
#define CHECK_GT(a, b) SHIM_CHECK_OP(a, b, >)
#define CHECK_GE(a, b) SHIM_CHECK_OP(a, b, >=)

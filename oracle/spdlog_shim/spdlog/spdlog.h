// TEST INFRASTRUCTURE ONLY.  Stand-in for the logging library the reference
// pins (spdlog v1.17.0, third-party/CMakeLists.txt:13-21), which is plumbing on
// this path: the free functions its headers call.  trace/debug/info are no-ops;
// warn/error/critical print the format string and its arguments to stderr when
// CSK_TEST_LOG is set in the environment (so a failing graph test can say why).
// No arithmetic of the reference depends on it.
#pragma once
#include <cstdlib>
#include <iostream>
namespace spdlog {
namespace shim {
template <typename T>
inline void put(const T& a) {
  if constexpr (requires(std::ostream& os, const T& x) { os << x; }) std::cerr << " [" << a << "]";
}
template <typename F, typename... A>
inline void print(const char* level, const F& fmt, const A&... args) {
  if (!std::getenv("CSK_TEST_LOG")) return;
  std::cerr << level << ": " << fmt;
  (put(args), ...);
  std::cerr << "\n";
}
}  // namespace shim
template <typename... A> inline void trace(A&&...) {}
template <typename... A> inline void debug(A&&...) {}
template <typename... A> inline void info(A&&...) {}
template <typename F, typename... A> inline void warn(const F& f, const A&... a) { shim::print("warn", f, a...); }
template <typename F, typename... A> inline void error(const F& f, const A&... a) { shim::print("error", f, a...); }
template <typename F, typename... A> inline void critical(const F& f, const A&... a) { shim::print("critical", f, a...); }
}  // namespace spdlog

// TEST INFRASTRUCTURE ONLY.  Stand-in for the logging library the reference
// pins (spdlog v1.17.0, third-party/CMakeLists.txt:13-21), which is plumbing on
// this path: the five free functions its headers call, as no-ops.  No
// arithmetic of the reference depends on it.
#pragma once
namespace spdlog {
template <typename... A> inline void trace(A&&...) {}
template <typename... A> inline void debug(A&&...) {}
template <typename... A> inline void info(A&&...) {}
template <typename... A> inline void warn(A&&...) {}
template <typename... A> inline void error(A&&...) {}
template <typename... A> inline void critical(A&&...) {}
}  // namespace spdlog

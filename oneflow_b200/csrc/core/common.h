#pragma once
#include <string>

#define OFC_API extern "C" __attribute__((visibility("default")))

namespace ofc {
inline std::string& last_error() {
  static thread_local std::string s;
  return s;
}
inline int fail(const std::string& m, int code = -1) {
  last_error() = m;
  return code;
}
}  // namespace ofc

// Minimal stand-ins for the logging / check macros Forward's creators use (easylogging's
// LOG(...) and the T_CHECK family), so the creator headers compile outside Forward's tree.
#pragma once

#include <iostream>
#include <sstream>

#ifndef LOG
namespace fwd {
namespace log_detail {
struct Line {
  explicit Line(bool on) : on_(on) {}
  ~Line() {
    if (on_) std::cerr << ss_.str() << std::endl;
  }
  template <typename T>
  Line& operator<<(const T& v) {
    if (on_) ss_ << v;
    return *this;
  }
  bool on_;
  std::ostringstream ss_;
};
inline bool Enabled(const char* level) { return level[0] == 'E'; }  // errors only
}  // namespace log_detail
}  // namespace fwd
#define LOG(level) ::fwd::log_detail::Line(::fwd::log_detail::Enabled(#level))
#endif

#ifndef T_CHECK
#define T_CHECK(cond)                                    \
  if (!(cond)) {                                         \
    LOG(ERROR) << "check failed: " #cond;                \
    return {};                                           \
  }
#define T_CHECK_LE(a, b) T_CHECK((a) <= (b))
#endif

// Minimal stand-ins for the logging / check macros Forward's creators use (easylogging's
// LOG(...) and the T_CHECK family), so the creator headers compile outside Forward's tree.
#pragma once

#include <cstdlib>
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
// Errors always; FWD_LOG_LEVEL=WARNING or INFO (read once) lets the quieter levels through too.
inline int Threshold() {
  static const int t = [] {
    const char* env = std::getenv("FWD_LOG_LEVEL");
    if (!env) return 2;
    return (env[0] == 'I' || env[0] == 'i') ? 0 : ((env[0] == 'W' || env[0] == 'w') ? 1 : 2);
  }();
  return t;
}
inline bool Enabled(const char* level) {
  const int rank = level[0] == 'I' ? 0 : (level[0] == 'W' ? 1 : 2);
  return rank >= Threshold();
}
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

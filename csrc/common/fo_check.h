// Argument checking for host code: FO_CHECK(cond, parts...) throws c10::Error (a Python
// RuntimeError) with the parts concatenated.
//
// The message is assembled with std::string / std::to_string on purpose.  TORCH_CHECK with
// several message parts formats through std::ostringstream inside the caller's object file;
// in processes where libc10.so (built with another toolchain) exports its own weak copies of
// libstdc++ stream symbols, those copies interpose on an extension built with the system
// compiler and the stream constructor crashes.  A single pre-built std::string avoids every
// stream symbol in this library.
#pragma once
#include <c10/util/Exception.h>

#include <string>
#include <type_traits>

namespace fo {
namespace detail {
inline void append(std::string& s, const char* v) { s += v; }
inline void append(std::string& s, const std::string& v) { s += v; }
inline void append(std::string& s, char v) { s += v; }
inline void append(std::string& s, bool v) { s += v ? "true" : "false"; }
template <class T>
typename std::enable_if<std::is_arithmetic<T>::value>::type append(std::string& s, T v) {
  s += std::to_string(v);
}
}  // namespace detail

template <class... Args>
std::string cat(const Args&... args) {
  std::string s;
  (void)std::initializer_list<int>{(detail::append(s, args), 0)...};
  return s;
}
}  // namespace fo

#define FO_CHECK(cond, ...)                                 \
  do {                                                      \
    if (!(cond)) {                                          \
      const std::string fo_msg__ = ::fo::cat(__VA_ARGS__);  \
      TORCH_CHECK(false, fo_msg__);                         \
    }                                                       \
  } while (0)

// Byte layout helpers for the plugin's engine blob.
//
// Wire format (must stay byte-compatible with Forward's
// source/trt_engine/trt_network_crt/plugins/common/serialize.hpp:41-118): a plain value is its
// raw bytes in host order; a vector is a size_t element count followed by the raw elements.
#pragma once

#include <cstddef>
#include <cstring>
#include <type_traits>
#include <vector>

namespace fwd {
namespace blob {

class Writer {
 public:
  explicit Writer(void* dst) : p_(static_cast<char*>(dst)) {}
  template <typename T>
  void value(const T& v) {
    static_assert(std::is_trivially_copyable<T>::value, "plain values only");
    std::memcpy(p_, &v, sizeof(T));
    p_ += sizeof(T);
  }
  void bytes(const void* src, size_t n) {
    if (n) std::memcpy(p_, src, n);
    p_ += n;
  }
  // count is in elements of `elem_size` bytes, as the reference's vector<T> writer stores it
  void counted(const void* src, size_t count, size_t elem_size) {
    value<size_t>(count);
    bytes(src, count * elem_size);
  }
  char* cursor() const { return p_; }

 private:
  char* p_;
};

class Reader {
 public:
  Reader(const void* src, size_t len) : p_(static_cast<const char*>(src)), left_(len) {}
  bool ok() const { return ok_; }
  size_t left() const { return left_; }
  template <typename T>
  bool value(T* out) {
    static_assert(std::is_trivially_copyable<T>::value, "plain values only");
    if (!ok_ || left_ < sizeof(T)) return ok_ = false;
    std::memcpy(out, p_, sizeof(T));
    p_ += sizeof(T);
    left_ -= sizeof(T);
    return true;
  }
  bool counted(std::vector<char>* out, size_t elem_size) {
    size_t count = 0;
    if (!value(&count)) return false;
    if (elem_size != 0 && count > left_ / elem_size) return ok_ = false;
    out->assign(p_, p_ + count * elem_size);
    p_ += count * elem_size;
    left_ -= count * elem_size;
    return true;
  }

 private:
  const char* p_;
  size_t left_;
  bool ok_{true};
};

}  // namespace blob
}  // namespace fwd

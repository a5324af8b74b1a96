// Little-endian byte writer / reader used by every binary format here. It
// plays the role of the reference's Sizer/Writer/Reader archivers
// (include/distributed/io.hpp:19-83, include/common/archiver.hpp:54-174):
// trivially copyable scalars are raw bytes, strings are u64 length + bytes,
// vectors are u64 count + elements.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace tnnb {

inline bool host_is_little_endian() {
  const uint16_t x = 1;
  return *reinterpret_cast<const uint8_t*>(&x) == 1;
}

template <typename T>
inline T byteswap(T v) {
  uint8_t b[sizeof(T)];
  std::memcpy(b, &v, sizeof(T));
  for (size_t i = 0; i < sizeof(T) / 2; ++i) std::swap(b[i], b[sizeof(T) - 1 - i]);
  std::memcpy(&v, b, sizeof(T));
  return v;
}

class ByteWriter {
 public:
  std::string buf;
  template <typename T>
  void put(T v) {
    static_assert(std::is_trivially_copyable<T>::value, "scalar expected");
    buf.append(reinterpret_cast<const char*>(&v), sizeof(T));
  }
  void raw(const void* p, size_t n) { buf.append(static_cast<const char*>(p), n); }
  void str(const std::string& s) {
    put<uint64_t>(s.size());
    buf.append(s);
  }
};

class ByteReader {
 public:
  ByteReader(const char* p, size_t n, bool swap = false) : p_(p), n_(n), swap_(swap) {}
  template <typename T>
  T get() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p_ + off_, sizeof(T));
    off_ += sizeof(T);
    return (swap_ && sizeof(T) > 1) ? byteswap(v) : v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    need(n);
    std::string s(p_ + off_, n);
    off_ += n;
    return s;
  }
  const char* take(size_t n) {
    need(n);
    const char* r = p_ + off_;
    off_ += n;
    return r;
  }
  size_t offset() const { return off_; }
  size_t remaining() const { return n_ - off_; }
  void set_swap(bool s) { swap_ = s; }

 private:
  void need(size_t n) const {
    if (n > n_ - off_) throw std::runtime_error("truncated buffer: need " + std::to_string(n) + " bytes at offset " + std::to_string(off_));
  }
  const char* p_;
  size_t n_;
  size_t off_ = 0;
  bool swap_;
};

}  // namespace tnnb

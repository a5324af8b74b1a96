// Element types shared by checkpoints, wire messages and kernels. The numeric
// values are part of the on-disk / on-wire formats (reference:
// include/type/type.hpp:115-128).
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace tnnb {

enum class DType : uint32_t {
  BYTE = 0, UINT8 = 1, INT8 = 2, BOOL = 3, FP16 = 4, BF16 = 5, FP32 = 6, FP64 = 7,
  INT32 = 8, INT64 = 9, SIZE_T = 10,
};

inline size_t dtype_size(DType t) {
  switch (t) {
    case DType::BYTE: case DType::UINT8: case DType::INT8: case DType::BOOL: return 1;
    case DType::FP16: case DType::BF16: return 2;
    case DType::FP32: case DType::INT32: return 4;
    case DType::FP64: case DType::INT64: case DType::SIZE_T: return 8;
  }
  throw std::runtime_error("unknown dtype code " + std::to_string(static_cast<uint32_t>(t)));
}

inline const char* dtype_name(DType t) {
  switch (t) {
    case DType::BYTE: return "BYTE"; case DType::UINT8: return "UINT8"; case DType::INT8: return "INT8";
    case DType::BOOL: return "BOOL"; case DType::FP16: return "FP16"; case DType::BF16: return "BF16";
    case DType::FP32: return "FP32"; case DType::FP64: return "FP64"; case DType::INT32: return "INT32";
    case DType::INT64: return "INT64"; case DType::SIZE_T: return "SIZE_T";
  }
  return "?";
}

inline DType dtype_from_name(const std::string& s) {
  static const char* names[] = {"BYTE", "UINT8", "INT8", "BOOL", "FP16", "BF16", "FP32", "FP64", "INT32", "INT64", "SIZE_T"};
  for (uint32_t i = 0; i < 11; ++i)
    if (s == names[i]) return static_cast<DType>(i);
  throw std::runtime_error("unknown dtype name " + s);
}

// bf16 <-> fp32 with round-to-nearest-even (reference software type: include/type/bf16.hpp:36-47).
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  __builtin_memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  __builtin_memcpy(&f, &u, 4);
  return f;
}

}  // namespace tnnb

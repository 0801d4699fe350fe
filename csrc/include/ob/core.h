// Core value types of the runtime: DType, Device, Layout and host float formats.
//
// Parity notes (paths are relative to the reference project):
//   DType set and sizes      include/orthon/core/dtype.h:6-23
//   Device parser            src/device/device.cpp:8-71
//   Layout contracts         include/orthon/core/layout.h:11-44, src/core/layout.cpp:9-105
//   f16/bf16 host converters src/core/float_formats.cpp:8-125
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace ob {

using Shape = std::vector<int64_t>;

enum class DType : uint8_t { F32 = 0, F64, F16, BF16, I32, I64, U8, I8, Bool, COUNT };

size_t dtype_size(DType d);
const char* dtype_name(DType d);
DType parse_dtype(const std::string& name);
inline bool dtype_is_floating(DType d) {
  return d == DType::F32 || d == DType::F64 || d == DType::F16 || d == DType::BF16;
}
inline bool dtype_is_low_precision(DType d) { return d == DType::F16 || d == DType::BF16; }

enum class DeviceType : uint8_t { CPU = 0, CUDA = 1 };

struct Device {
  DeviceType type = DeviceType::CPU;
  int index = 0;
  Device() = default;
  Device(DeviceType t, int i) : type(t), index(i) {}
  bool is_cuda() const { return type == DeviceType::CUDA; }
  bool is_cpu() const { return type == DeviceType::CPU; }
  bool operator==(const Device& o) const { return type == o.type && index == o.index; }
  bool operator!=(const Device& o) const { return !(*this == o); }
  std::string str() const;
  // Accepts exactly "cpu", "cuda" (meaning cuda:0) or "cuda:N" with decimal N.
  static Device parse(const std::string& text);
};

// Immutable shape/strides/offset triple with overflow-checked element counts.
// Strides are in elements and never negative.
class Layout {
 public:
  Layout() : numel_(1) {}
  explicit Layout(Shape shape);
  Layout(Shape shape, Shape strides, int64_t offset);

  const Shape& shape() const { return shape_; }
  const Shape& strides() const { return strides_; }
  int64_t offset() const { return offset_; }
  int64_t numel() const { return numel_; }
  int ndim() const { return static_cast<int>(shape_.size()); }
  // Size-1 dimensions never break contiguity.
  bool is_contiguous() const;
  // One past the largest element offset touched (0 for empty tensors), offset included.
  int64_t span_end() const;
  void validate_bounds(size_t capacity_bytes, size_t element_size) const;

  static Shape contiguous_strides(const Shape& shape);
  static int64_t checked_numel(const Shape& shape);

 private:
  Shape shape_;
  Shape strides_;
  int64_t offset_ = 0;
  int64_t numel_ = 1;
};

// NumPy-style broadcast of two shapes; a size-1 extent stretches to the other
// extent, including 0.  (reference: src/core/broadcast.cpp:11-31)
Shape broadcast_shapes(const Shape& a, const Shape& b);
std::string shape_str(const Shape& s);

// Host conversions, round-to-nearest-even.  f16 keeps NaN payload bits, bf16
// quiets NaNs; subnormals are handled exactly.
uint16_t f32_to_f16(float v);
float f16_to_f32(uint16_t h);
uint16_t f32_to_bf16(float v);
float bf16_to_f32(uint16_t b);

double load_as_double(const void* p, DType d);
void store_from_double(void* p, DType d, double v);

#define OB_CHECK(cond, msg)                                   \
  do {                                                        \
    if (!(cond)) throw std::runtime_error(std::string(msg));  \
  } while (0)
#define OB_CHECK_ARG(cond, msg)                                  \
  do {                                                           \
    if (!(cond)) throw std::invalid_argument(std::string(msg));  \
  } while (0)

// Debug channel gated by ORTHON_DEBUG_DEVICE=1 (reference: src/utils/logging.cpp:7-22).
bool debug_device_enabled();
void debug_device_log(const std::string& line);

}  // namespace ob

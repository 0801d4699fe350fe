// DType / Device / Layout / broadcast / host float formats.
#include "ob/core.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <sstream>

namespace ob {

size_t dtype_size(DType d) {
  switch (d) {
    case DType::F32: return 4;
    case DType::F64: return 8;
    case DType::F16: return 2;
    case DType::BF16: return 2;
    case DType::I32: return 4;
    case DType::I64: return 8;
    case DType::U8: return 1;
    case DType::I8: return 1;
    case DType::Bool: return 1;
    default: break;
  }
  throw std::invalid_argument("dtype_size: unknown dtype");
}

const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "float32";
    case DType::F64: return "float64";
    case DType::F16: return "float16";
    case DType::BF16: return "bfloat16";
    case DType::I32: return "int32";
    case DType::I64: return "int64";
    case DType::U8: return "uint8";
    case DType::I8: return "int8";
    case DType::Bool: return "bool";
    default: break;
  }
  return "unknown";
}

DType parse_dtype(const std::string& name) {
  for (int i = 0; i < static_cast<int>(DType::COUNT); ++i) {
    if (name == dtype_name(static_cast<DType>(i))) return static_cast<DType>(i);
  }
  throw std::invalid_argument("unknown dtype '" + name + "'");
}

std::string Device::str() const {
  if (type == DeviceType::CPU) return "cpu";
  return "cuda:" + std::to_string(index);
}

Device Device::parse(const std::string& text) {
  if (text == "cpu") return Device(DeviceType::CPU, 0);
  if (text == "cuda") return Device(DeviceType::CUDA, 0);
  const std::string prefix = "cuda:";
  if (text.rfind(prefix, 0) == 0 && text.size() > prefix.size()) {
    const std::string digits = text.substr(prefix.size());
    if (digits.size() > 9) throw std::invalid_argument("invalid device string '" + text + "'");
    for (char c : digits) {
      if (c < '0' || c > '9') throw std::invalid_argument("invalid device string '" + text + "'");
    }
    return Device(DeviceType::CUDA, std::stoi(digits));
  }
  throw std::invalid_argument("invalid device string '" + text + "'");
}

int64_t Layout::checked_numel(const Shape& shape) {
  int64_t n = 1;
  for (int64_t d : shape) {
    if (d < 0) throw std::invalid_argument("shape extents must be non-negative");
    if (d != 0 && n > std::numeric_limits<int64_t>::max() / d)
      throw std::overflow_error("shape element count overflows int64");
    n *= d;
  }
  return n;
}

Shape Layout::contiguous_strides(const Shape& shape) {
  Shape st(shape.size());
  int64_t run = 1;
  for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
    st[i] = run;
    run *= (shape[i] == 0 ? 1 : shape[i]);
  }
  return st;
}

Layout::Layout(Shape shape) : shape_(std::move(shape)) {
  numel_ = checked_numel(shape_);
  strides_ = contiguous_strides(shape_);
}

Layout::Layout(Shape shape, Shape strides, int64_t offset)
    : shape_(std::move(shape)), strides_(std::move(strides)), offset_(offset) {
  if (shape_.size() != strides_.size()) throw std::invalid_argument("layout: shape/strides rank mismatch");
  if (offset_ < 0) throw std::invalid_argument("layout: negative offset");
  for (int64_t s : strides_)
    if (s < 0) throw std::invalid_argument("layout: negative strides are not supported");
  numel_ = checked_numel(shape_);
}

bool Layout::is_contiguous() const {
  int64_t run = 1;
  for (int i = ndim() - 1; i >= 0; --i) {
    if (shape_[i] == 1) continue;
    if (shape_[i] == 0) return true;
    if (strides_[i] != run) return false;
    run *= shape_[i];
  }
  return true;
}

int64_t Layout::span_end() const {
  if (numel_ == 0) return 0;
  int64_t last = offset_;
  for (int i = 0; i < ndim(); ++i) {
    const int64_t ext = shape_[i] - 1;
    if (ext != 0 && strides_[i] != 0) {
      if (strides_[i] > (std::numeric_limits<int64_t>::max() - last) / ext)
        throw std::overflow_error("layout: storage span overflows int64");
      last += ext * strides_[i];
    }
  }
  return last + 1;
}

void Layout::validate_bounds(size_t capacity_bytes, size_t element_size) const {
  const int64_t end = span_end();
  if (end == 0) return;
  if (static_cast<uint64_t>(end) > capacity_bytes / element_size)
    throw std::out_of_range("layout: view exceeds the bounds of its buffer");
}

Shape broadcast_shapes(const Shape& a, const Shape& b) {
  const size_t n = std::max(a.size(), b.size());
  Shape out(n);
  for (size_t i = 0; i < n; ++i) {
    const int64_t da = i < n - a.size() ? 1 : a[i - (n - a.size())];
    const int64_t db = i < n - b.size() ? 1 : b[i - (n - b.size())];
    if (da == db) out[i] = da;
    else if (da == 1) out[i] = db;
    else if (db == 1) out[i] = da;
    else
      throw std::invalid_argument("shapes " + shape_str(a) + " and " + shape_str(b) +
                                  " are not broadcastable");
  }
  return out;
}

std::string shape_str(const Shape& s) {
  std::ostringstream os;
  os << "[";
  for (size_t i = 0; i < s.size(); ++i) os << (i ? ", " : "") << s[i];
  os << "]";
  return os.str();
}

// ---------------------------------------------------------------- float formats
static inline uint32_t f32_bits(float v) { uint32_t u; std::memcpy(&u, &v, 4); return u; }
static inline float bits_f32(uint32_t u) { float v; std::memcpy(&v, &u, 4); return v; }

uint16_t f32_to_f16(float v) {
  const uint32_t x = f32_bits(v);
  const uint16_t sign = static_cast<uint16_t>((x >> 16) & 0x8000u);
  const uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) {  // inf / nan
    if (absx == 0x7f800000u) return sign | 0x7c00u;
    uint16_t payload = static_cast<uint16_t>((absx >> 13) & 0x3ffu);
    if (payload == 0) payload = 1;  // keep it a NaN when only low payload bits were set
    return sign | 0x7c00u | payload;
  }
  const int32_t exp = static_cast<int32_t>(absx >> 23) - 127 + 15;
  uint32_t mant = absx & 0x7fffffu;
  if (exp >= 31) return sign | 0x7c00u;  // overflow to inf
  if (exp <= 0) {                        // subnormal or zero
    if (exp < -10) return sign;
    mant |= 0x800000u;
    const int shift = 14 - exp;  // bits dropped
    const uint32_t half = 1u << (shift - 1);
    const uint32_t rem = mant & ((1u << shift) - 1);
    uint32_t r = mant >> shift;
    if (rem > half || (rem == half && (r & 1u))) ++r;
    return sign | static_cast<uint16_t>(r);
  }
  uint32_t r = (static_cast<uint32_t>(exp) << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;  // may carry into exponent/inf, which is right
  return sign | static_cast<uint16_t>(r);
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t mant = h & 0x3ffu;
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (mant << 13));
  if (exp == 0) {
    if (mant == 0) return bits_f32(sign);
    int e = -1;
    do { ++e; mant <<= 1; } while ((mant & 0x400u) == 0);
    mant &= 0x3ffu;
    return bits_f32(sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | (mant << 13));
  }
  return bits_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

uint16_t f32_to_bf16(float v) {
  const uint32_t x = f32_bits(v);
  if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x0040u);  // quiet NaN
  const uint32_t lsb = (x >> 16) & 1u;
  return static_cast<uint16_t>((x + 0x7fffu + lsb) >> 16);
}

float bf16_to_f32(uint16_t b) { return bits_f32(static_cast<uint32_t>(b) << 16); }

double load_as_double(const void* p, DType d) {
  switch (d) {
    case DType::F32: { float v; std::memcpy(&v, p, 4); return v; }
    case DType::F64: { double v; std::memcpy(&v, p, 8); return v; }
    case DType::F16: { uint16_t v; std::memcpy(&v, p, 2); return f16_to_f32(v); }
    case DType::BF16: { uint16_t v; std::memcpy(&v, p, 2); return bf16_to_f32(v); }
    case DType::I32: { int32_t v; std::memcpy(&v, p, 4); return v; }
    case DType::I64: { int64_t v; std::memcpy(&v, p, 8); return static_cast<double>(v); }
    case DType::U8: return *static_cast<const uint8_t*>(p);
    case DType::I8: return *static_cast<const int8_t*>(p);
    case DType::Bool: return *static_cast<const uint8_t*>(p) ? 1.0 : 0.0;
    default: break;
  }
  throw std::invalid_argument("load_as_double: unknown dtype");
}

void store_from_double(void* p, DType d, double v) {
  switch (d) {
    case DType::F32: { float x = static_cast<float>(v); std::memcpy(p, &x, 4); return; }
    case DType::F64: { std::memcpy(p, &v, 8); return; }
    case DType::F16: { uint16_t x = f32_to_f16(static_cast<float>(v)); std::memcpy(p, &x, 2); return; }
    case DType::BF16: { uint16_t x = f32_to_bf16(static_cast<float>(v)); std::memcpy(p, &x, 2); return; }
    case DType::I32: { int32_t x = static_cast<int32_t>(v); std::memcpy(p, &x, 4); return; }
    case DType::I64: { int64_t x = static_cast<int64_t>(v); std::memcpy(p, &x, 8); return; }
    case DType::U8: { *static_cast<uint8_t*>(p) = static_cast<uint8_t>(v); return; }
    case DType::I8: { *static_cast<int8_t*>(p) = static_cast<int8_t>(v); return; }
    case DType::Bool: { *static_cast<uint8_t*>(p) = (v != 0.0) ? 1 : 0; return; }
    default: break;
  }
  throw std::invalid_argument("store_from_double: unknown dtype");
}

bool debug_device_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("ORTHON_DEBUG_DEVICE");
    return v != nullptr && std::string(v) == "1";
  }();
  return on;
}

void debug_device_log(const std::string& line) {
  if (debug_device_enabled()) std::fprintf(stderr, "[orthon:device] %s\n", line.c_str());
}

}  // namespace ob

// Layout arithmetic, broadcasting, dtypes, the device parser and the host float formats, one
// contract per case.  (reference project: tests/cpp/test_tensor_core.cpp, test_float_formats.cpp,
// test_device_guard.cpp)
#include <cmath>
#include <cstring>
#include <limits>

#include "check.h"
#include "ob/core.h"

using namespace ob;

namespace {
uint32_t bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
float from_bits(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
}  // namespace

TEST(layout_default_is_a_scalar_like_single_element) {
  Layout l;
  CHECK_EQ(l.numel(), 1);
  CHECK_EQ(l.ndim(), 0);
  CHECK(l.is_contiguous());
}
TEST(layout_contiguous_strides_are_row_major) {
  CHECK(Layout::contiguous_strides({2, 3, 4}) == (Shape{12, 4, 1}));
  CHECK(Layout::contiguous_strides({5}) == (Shape{1}));
  CHECK(Layout::contiguous_strides({}) == (Shape{}));
}
TEST(layout_from_shape_is_packed) {
  Layout l(Shape{2, 3});
  CHECK(l.strides() == (Shape{3, 1}));
  CHECK_EQ(l.numel(), 6);
  CHECK_EQ(l.offset(), 0);
  CHECK_EQ(l.span_end(), 6);
}
TEST(layout_rejects_negative_extents) { CHECK_THROWS(Layout(Shape{2, -1})); }
TEST(layout_rejects_negative_strides) { CHECK_THROWS(Layout(Shape{2, 2}, Shape{-2, 1}, 0)); }
TEST(layout_rejects_negative_offset) { CHECK_THROWS(Layout(Shape{2}, Shape{1}, -1)); }
TEST(layout_rejects_rank_mismatch) { CHECK_THROWS(Layout(Shape{2, 2}, Shape{1}, 0)); }
TEST(layout_numel_overflow_is_detected) {
  CHECK_THROWS(Layout::checked_numel({int64_t(1) << 40, int64_t(1) << 40}));
  CHECK_EQ(Layout::checked_numel({0, int64_t(1) << 62}), 0);
}
TEST(layout_size_one_dimensions_never_break_contiguity) {
  CHECK(Layout(Shape{1, 4}, Shape{99, 1}, 0).is_contiguous());
  CHECK(Layout(Shape{3, 1, 4}, Shape{4, 7, 1}, 0).is_contiguous());
  CHECK(!Layout(Shape{3, 4}, Shape{1, 3}, 0).is_contiguous());
}
TEST(layout_empty_tensors_are_contiguous_and_span_nothing) {
  Layout l(Shape{0, 5});
  CHECK(l.is_contiguous());
  CHECK_EQ(l.numel(), 0);
  CHECK_EQ(l.span_end(), 0);
}
TEST(layout_span_of_a_strided_view_includes_the_offset) {
  Layout l(Shape{2, 2}, Shape{1, 3}, 4);  // transposed corner of a [*, 3] matrix
  CHECK_EQ(l.span_end(), 4 + 1 + 3 + 1);
}
TEST(layout_bounds_are_checked_against_capacity) {
  Layout ok(Shape{2, 3}, Shape{3, 1}, 2);
  ok.validate_bounds(8 * 4, 4);
  CHECK_THROWS(ok.validate_bounds(7 * 4, 4));
  Layout(Shape{0}, Shape{1}, 100).validate_bounds(0, 4);  // an empty view touches nothing
}
TEST(broadcast_equal_shapes) { CHECK(broadcast_shapes({2, 3}, {2, 3}) == (Shape{2, 3})); }
TEST(broadcast_prepends_missing_dimensions) { CHECK(broadcast_shapes({4}, {2, 3, 4}) == (Shape{2, 3, 4})); }
TEST(broadcast_stretches_ones_both_ways) { CHECK(broadcast_shapes({3, 1}, {1, 4}) == (Shape{3, 4})); }
TEST(broadcast_stretches_one_to_zero) { CHECK(broadcast_shapes({1, 3}, {0, 3}) == (Shape{0, 3})); }
TEST(broadcast_with_a_scalar_like_shape) { CHECK(broadcast_shapes({}, {2, 2}) == (Shape{2, 2})); }
TEST(broadcast_rejects_incompatible_extents) {
  CHECK_THROWS(broadcast_shapes({2, 3}, {3, 2}));
  CHECK_THROWS(broadcast_shapes({0}, {2}));
}
TEST(shape_text) {
  CHECK_EQ(shape_str({2, 3}), std::string("[2, 3]"));
  CHECK_EQ(shape_str({}), std::string("[]"));
}
TEST(dtype_sizes) {
  CHECK_EQ(dtype_size(DType::F32), 4u); CHECK_EQ(dtype_size(DType::F64), 8u); CHECK_EQ(dtype_size(DType::F16), 2u);
  CHECK_EQ(dtype_size(DType::BF16), 2u); CHECK_EQ(dtype_size(DType::I32), 4u); CHECK_EQ(dtype_size(DType::I64), 8u);
  CHECK_EQ(dtype_size(DType::U8), 1u); CHECK_EQ(dtype_size(DType::I8), 1u); CHECK_EQ(dtype_size(DType::Bool), 1u);
}
TEST(dtype_names_round_trip) {
  for (int i = 0; i < static_cast<int>(DType::COUNT); ++i) {
    const DType d = static_cast<DType>(i);
    CHECK(parse_dtype(dtype_name(d)) == d);
  }
  CHECK_THROWS(parse_dtype("float8"));
  CHECK_THROWS(parse_dtype(""));
}
TEST(dtype_classes) {
  CHECK(dtype_is_floating(DType::BF16) && dtype_is_floating(DType::F64) && !dtype_is_floating(DType::I64) && !dtype_is_floating(DType::Bool));
  CHECK(dtype_is_low_precision(DType::F16) && !dtype_is_low_precision(DType::F32));
}
TEST(device_parser_accepts_the_three_spellings) {
  CHECK(Device::parse("cpu") == Device(DeviceType::CPU, 0));
  CHECK(Device::parse("cuda") == Device(DeviceType::CUDA, 0));
  CHECK(Device::parse("cuda:3") == Device(DeviceType::CUDA, 3));
  CHECK_EQ(Device::parse("cuda:12").str(), std::string("cuda:12"));
  CHECK_EQ(Device().str(), std::string("cpu"));
}
TEST(device_parser_is_strict) {
  for (const char* bad : {"", "CPU", "cpu:0", "cuda:", "cuda:-1", "cuda:1x", "cuda: 1", " cuda", "gpu", "cuda:+1", "cuda:0x1"})
    CHECK_THROWS(Device::parse(bad));
}
TEST(device_equality) {
  CHECK(Device(DeviceType::CUDA, 1) != Device(DeviceType::CUDA, 2));
  CHECK(Device(DeviceType::CUDA, 0) != Device(DeviceType::CPU, 0));
  CHECK(Device(DeviceType::CUDA, 0).is_cuda() && Device().is_cpu());
}
TEST(f16_exact_values_round_trip) {
  for (float v : {0.0f, 1.0f, -2.0f, 0.5f, 65504.0f, 6.103515625e-05f /* smallest normal */, 5.9604644775390625e-08f /* smallest subnormal */})
    CHECK_EQ(f16_to_f32(f32_to_f16(v)), v);
  CHECK_EQ(f32_to_f16(-0.0f), 0x8000);
}
TEST(f16_rounds_to_nearest_even) {
  CHECK_EQ(f32_to_f16(1.0f + 0.00048828125f), 0x3C00);          // exactly half way between 1 and the next value: even wins
  CHECK_EQ(f32_to_f16(1.0f + 3 * 0.00048828125f), 0x3C02);      // half way, odd below: rounds up to even
  CHECK_EQ(f32_to_f16(1.0f + 0.0005f), 0x3C01);
}
TEST(f16_overflow_and_underflow) {
  CHECK_EQ(f32_to_f16(65520.0f), 0x7C00);                        // rounds to infinity
  CHECK_EQ(f32_to_f16(-1e9f), 0xFC00);
  CHECK_EQ(f32_to_f16(1e-10f), 0x0000);
  CHECK_EQ(f32_to_f16(2.98023223876953125e-08f), 0x0000);        // half of the smallest subnormal: ties to even (zero)
  CHECK_EQ(f32_to_f16(4.5e-08f), 0x0001);
}
TEST(f16_keeps_nan_payload_and_infinities) {
  CHECK(std::isinf(f16_to_f32(0x7C00)) && f16_to_f32(0xFC00) < 0);
  const uint16_t h = f32_to_f16(from_bits(0x7FC12000u));
  CHECK((h & 0x7C00) == 0x7C00 && (h & 0x03FF) != 0);
  CHECK(std::isnan(f16_to_f32(0x7E01)));
  CHECK_EQ(bits(f16_to_f32(0x7E01)) & 0x007FE000u, (0x0201u << 13));
}
TEST(bf16_is_the_rounded_upper_half) {
  CHECK_EQ(f32_to_bf16(1.0f), 0x3F80);
  CHECK_EQ(bf16_to_f32(0x3F80), 1.0f);
  CHECK_EQ(f32_to_bf16(from_bits(0x3F808000u)), 0x3F80);         // tie, even below
  CHECK_EQ(f32_to_bf16(from_bits(0x3F818000u)), 0x3F82);         // tie, odd below: up
  CHECK_EQ(f32_to_bf16(from_bits(0x3F808001u)), 0x3F81);
  CHECK_EQ(f32_to_bf16(-0.0f), 0x8000);
}
TEST(bf16_rounding_can_reach_infinity_and_quiets_nan) {
  CHECK_EQ(f32_to_bf16(std::numeric_limits<float>::max()), 0x7F80);
  CHECK_EQ(f32_to_bf16(std::numeric_limits<float>::infinity()), 0x7F80);
  const uint16_t n = f32_to_bf16(from_bits(0x7F800001u));        // a signalling NaN whose payload sits in the dropped half
  CHECK((n & 0x7F80) == 0x7F80 && (n & 0x007F) != 0);
  CHECK(std::isnan(bf16_to_f32(n)));
}
TEST(bf16_keeps_float32_subnormal_range) {
  const float tiny = from_bits(0x00010000u);
  CHECK_EQ(bf16_to_f32(f32_to_bf16(tiny)), tiny);
}
TEST(scalar_load_store_by_dtype) {
  unsigned char cell[8];
  for (int i = 0; i < static_cast<int>(DType::COUNT); ++i) {
    const DType d = static_cast<DType>(i);
    store_from_double(cell, d, 3.0);
    CHECK_EQ(load_as_double(cell, d), d == DType::Bool ? 1.0 : 3.0);
  }
  store_from_double(cell, DType::U8, 255.0);
  CHECK_EQ(load_as_double(cell, DType::U8), 255.0);
  store_from_double(cell, DType::I8, -128.0);
  CHECK_EQ(load_as_double(cell, DType::I8), -128.0);
  store_from_double(cell, DType::F16, 0.1);
  CHECK_NEAR(load_as_double(cell, DType::F16), 0.1, 1e-4);
}

// Core value types: DType, Device, Layout, broadcast, host float formats.
// (reference project: tests/cpp core domain - layout, dtype, device, float format cases)
#include <cmath>
#include <limits>

#include "check.h"
#include "ob/core.h"

using namespace ob;

TEST(dtype_sizes_names_and_parsing) {
  CHECK_EQ(dtype_size(DType::F32), 4u);
  CHECK_EQ(dtype_size(DType::F64), 8u);
  CHECK_EQ(dtype_size(DType::F16), 2u);
  CHECK_EQ(dtype_size(DType::BF16), 2u);
  CHECK_EQ(dtype_size(DType::I32), 4u);
  CHECK_EQ(dtype_size(DType::I64), 8u);
  CHECK_EQ(dtype_size(DType::U8), 1u);
  CHECK_EQ(dtype_size(DType::I8), 1u);
  CHECK_EQ(dtype_size(DType::Bool), 1u);
  for (int d = 0; d < static_cast<int>(DType::COUNT); ++d)
    CHECK(parse_dtype(dtype_name(static_cast<DType>(d))) == static_cast<DType>(d));
  CHECK_THROWS(parse_dtype("float128"));
  CHECK(dtype_is_floating(DType::BF16) && !dtype_is_floating(DType::I64) && !dtype_is_floating(DType::Bool));
}

TEST(device_parser_is_strict) {
  CHECK(Device::parse("cpu") == Device(DeviceType::CPU, 0));
  CHECK(Device::parse("cuda") == Device(DeviceType::CUDA, 0));
  CHECK(Device::parse("cuda:3") == Device(DeviceType::CUDA, 3));
  CHECK_EQ(Device::parse("cuda:12").str(), std::string("cuda:12"));
  CHECK_EQ(Device().str(), std::string("cpu"));
  for (const char* bad : {"", "gpu", "cuda:", "cuda:-1", "cuda:1x", "CPU", " cpu", "cuda: 1", "cpu:0x"}) CHECK_THROWS(Device::parse(bad));
}

TEST(layout_contiguous_strides_and_numel) {
  const Layout l(Shape{2, 3, 4});
  CHECK(l.strides() == (Shape{12, 4, 1}));
  CHECK_EQ(l.numel(), 24);
  CHECK_EQ(l.offset(), 0);
  CHECK(l.is_contiguous());
  CHECK_EQ(l.span_end(), 24);
  CHECK_EQ(Layout(Shape{}).numel(), 1);        // rank 0 holds one element
  CHECK_EQ(Layout(Shape{0, 5}).numel(), 0);
  CHECK_EQ(Layout(Shape{0, 5}).span_end(), 0);  // an empty tensor touches nothing
}

TEST(layout_contiguity_ignores_unit_dimensions) {
  CHECK(Layout(Shape{1, 4}, Shape{999, 1}, 0).is_contiguous());
  CHECK(Layout(Shape{3, 1, 4}, Shape{4, 77, 1}, 0).is_contiguous());
  CHECK(!Layout(Shape{3, 4}, Shape{1, 3}, 0).is_contiguous());  // transposed
  CHECK(!Layout(Shape{3, 4}, Shape{8, 1}, 0).is_contiguous());  // padded rows
}

TEST(layout_views_offsets_and_bounds) {
  const Layout v(Shape{2, 2}, Shape{4, 1}, 5);  // a 2x2 window of a 4-wide matrix
  CHECK_EQ(v.span_end(), 5 + 4 + 1 + 1);
  v.validate_bounds(11 * 4, 4);
  CHECK_THROWS(v.validate_bounds(10 * 4, 4));
  CHECK_THROWS(Layout(Shape{2, 2}, Shape{-1, 1}, 0));  // negative strides are not representable
  CHECK_THROWS(Layout(Shape{2, 2}, Shape{1}, 0));       // rank mismatch
  CHECK_THROWS(Layout(Shape{2, -2}));
  CHECK_THROWS(Layout(Shape{2, 2}, Shape{2, 1}, -1));
}

TEST(layout_element_count_overflow_is_checked) {
  const int64_t big = int64_t(1) << 40;
  CHECK_THROWS(Layout::checked_numel(Shape{big, big}));
  CHECK_THROWS(Layout(Shape{big, big, 4}));
  CHECK_EQ(Layout::checked_numel(Shape{big, 0, big}), 0);
}

TEST(broadcast_shapes_follow_numpy) {
  CHECK(broadcast_shapes(Shape{2, 3}, Shape{3}) == (Shape{2, 3}));
  CHECK(broadcast_shapes(Shape{4, 1, 3}, Shape{5, 1}) == (Shape{4, 5, 3}));
  CHECK(broadcast_shapes(Shape{}, Shape{2}) == (Shape{2}));
  CHECK(broadcast_shapes(Shape{1}, Shape{0}) == (Shape{0}));  // size 1 stretches to 0 as well
  CHECK(broadcast_shapes(Shape{3, 1}, Shape{1, 0}) == (Shape{3, 0}));
  CHECK_THROWS(broadcast_shapes(Shape{2, 3}, Shape{4}));
  CHECK_THROWS(broadcast_shapes(Shape{2}, Shape{0}));
}

TEST(float16_round_to_nearest_even_and_specials) {
  CHECK_EQ(f32_to_f16(1.0f), 0x3C00);
  CHECK_EQ(f32_to_f16(-2.0f), 0xC000);
  CHECK_EQ(f32_to_f16(65504.0f), 0x7BFF);
  CHECK_EQ(f32_to_f16(65520.0f), 0x7C00);                                 // rounds up to infinity
  CHECK_EQ(f32_to_f16(std::numeric_limits<float>::infinity()), 0x7C00);
  CHECK_EQ(f32_to_f16(5.9604645e-8f), 0x0001);                            // smallest subnormal
  CHECK_EQ(f32_to_f16(2.9802322e-8f), 0x0000);                            // tie to even: zero
  CHECK_EQ(f32_to_f16(1.0f + 1.0f / 2048.0f), 0x3C00);                    // tie to even (down)
  CHECK_EQ(f32_to_f16(1.0f + 3.0f / 2048.0f), 0x3C02);                    // tie to even (up)
  CHECK_EQ(f32_to_f16(-0.0f), 0x8000);
  CHECK(std::isnan(f16_to_f32(f32_to_f16(std::nanf("")))));
  for (uint32_t h = 0; h < 0x10000; ++h) {                                // every half value survives a round trip
    const uint16_t half = static_cast<uint16_t>(h);
    const float f = f16_to_f32(half);
    if (std::isnan(f)) continue;
    CHECK_EQ(f32_to_f16(f), half);
  }
}

TEST(bfloat16_round_to_nearest_even_and_specials) {
  CHECK_EQ(f32_to_bf16(1.0f), 0x3F80);
  CHECK_EQ(f32_to_bf16(-1.5f), 0xBFC0);
  CHECK_EQ(f32_to_bf16(1.0f + 1.0f / 256.0f), 0x3F80);   // tie to even (down)
  CHECK_EQ(f32_to_bf16(1.0f + 3.0f / 256.0f), 0x3F82);   // tie to even (up)
  CHECK_EQ(f32_to_bf16(std::numeric_limits<float>::infinity()), 0x7F80);
  CHECK_EQ(f32_to_bf16(3.4e38f), 0x7F80);                 // above the largest finite bfloat16
  const uint16_t nan_bits = f32_to_bf16(std::nanf(""));
  CHECK((nan_bits & 0x7F80) == 0x7F80 && (nan_bits & 0x007F) != 0 && (nan_bits & 0x0040) != 0);  // quiet NaN
  for (uint32_t b = 0; b < 0x10000; ++b) {
    const uint16_t bits = static_cast<uint16_t>(b);
    const float f = bf16_to_f32(bits);
    if (std::isnan(f)) continue;
    CHECK_EQ(f32_to_bf16(f), bits);
  }
}

TEST(typed_load_and_store_through_double) {
  alignas(8) unsigned char cell[8];
  const DType all[] = {DType::F32, DType::F64, DType::F16, DType::BF16, DType::I32, DType::I64, DType::U8, DType::I8, DType::Bool};
  for (DType d : all) {
    store_from_double(cell, d, 1.0);
    CHECK_NEAR(load_as_double(cell, d), 1.0, 0.0);
  }
  store_from_double(cell, DType::I8, -7.0);
  CHECK_NEAR(load_as_double(cell, DType::I8), -7.0, 0.0);
  store_from_double(cell, DType::F16, 0.1);
  CHECK_NEAR(load_as_double(cell, DType::F16), 0.1, 1e-4);
  store_from_double(cell, DType::Bool, 5.0);
  CHECK_NEAR(load_as_double(cell, DType::Bool), 1.0, 0.0);
}

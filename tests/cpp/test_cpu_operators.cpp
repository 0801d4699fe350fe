// Semantic operators on the CPU backend through the C++ API: values, validation and the
// messages callers rely on.  (reference project: tests/cpp/test_ops_binary.cpp, test_ops_matmul.cpp,
// test_ops_reduce.cpp, test_ops_scalar.cpp, test_ops_shape.cpp, test_ops_to.cpp, test_ops_unary.cpp,
// test_indexing.cpp, test_reduction_subsystem.cpp)
#include <cmath>
#include <limits>
#include <vector>

#include "check.h"
#include "ob/ops.h"
#include "ob/tensor.h"

using namespace ob;

namespace {
const Device kCpu;
Tensor make(const Shape& shape, std::initializer_list<double> v, DType dt = DType::F32) {
  Tensor t = Tensor::empty(shape, dt, kCpu);
  int64_t i = 0;
  for (double x : v) ops::write_scalar(t, i++, x);
  return t;
}
std::vector<double> vals(const Tensor& t) {
  Tensor c = ops::contiguous(t);
  std::vector<double> out;
  for (int64_t i = 0; i < c.numel(); ++i) out.push_back(ops::read_scalar(c, i));
  return out;
}
using V = std::vector<double>;
}  // namespace

TEST(cpu_add_broadcasts_rows_and_columns) {
  Tensor a = make({2, 3}, {1, 2, 3, 4, 5, 6});
  CHECK(vals(ops::add(a, make({3}, {10, 20, 30}))) == (V{11, 22, 33, 14, 25, 36}));
  CHECK(vals(ops::add(a, make({2, 1}, {100, 200}))) == (V{101, 102, 103, 204, 205, 206}));
  CHECK(ops::add(make({3, 1}, {1, 2, 3}), make({1, 2}, {10, 20})).shape() == (Shape{3, 2}));
}
TEST(cpu_sub_and_div_are_composed) {
  CHECK(vals(ops::sub(make({2}, {5, 7}), make({2}, {1, 2}))) == (V{4, 5}));
  CHECK(vals(ops::div(make({2}, {6, 9}), make({2}, {2, 3}))) == (V{3, 3}));
  CHECK(std::isinf(vals(ops::div(make({1}, {1}), make({1}, {0})))[0]));
}
TEST(cpu_binary_validation) {
  CHECK_THROWS(ops::add(make({2}, {1, 2}), make({3}, {1, 2, 3})));
  CHECK_THROWS_WITH(ops::add(make({2}, {1, 2}), make({2}, {1, 2}, DType::F64)), "dtype mismatch");
  CHECK_THROWS(ops::mul(make({2}, {1, 2}, DType::I32), make({2}, {1, 2}, DType::I32)));  // compute dtypes are floating
}
TEST(cpu_float64_arithmetic_keeps_precision) {
  Tensor a = make({1}, {1.0}, DType::F64), b = make({1}, {1e-12}, DType::F64);
  CHECK(vals(ops::add(a, b))[0] != 1.0);
  CHECK(ops::add(a, b).dtype() == DType::F64);
}
TEST(cpu_scalar_forms) {
  Tensor a = make({3}, {1, 2, 3});
  CHECK(vals(ops::add_scalar(a, 0.5)) == (V{1.5, 2.5, 3.5}));
  CHECK(vals(ops::mul_scalar(a, -2)) == (V{-2, -4, -6}));
  CHECK(ops::mul_scalar(make({0}, {}), 3).numel() == 0);
}
TEST(cpu_inplace_add_and_mul) {
  Tensor a = make({3}, {1, 2, 3});
  ops::add_(a, make({3}, {10, 10, 10}), 0.5);
  CHECK(vals(a) == (V{6, 7, 8}));
  ops::mul_(a, 2.0);
  CHECK(vals(a) == (V{12, 14, 16}));
  ops::add_(a, make({1}, {1}), 1.0);  // the right operand may broadcast
  CHECK(vals(a) == (V{13, 15, 17}));
  CHECK_THROWS(ops::add_(a, make({2, 3}, {1, 2, 3, 4, 5, 6}), 1.0));  // the left one may not grow
}
TEST(cpu_inplace_rejects_partial_overlap_but_allows_identity) {
  Tensor base = make({4}, {1, 2, 3, 4});
  Tensor left = ops::slice(base, 0, 0, 3), right = ops::slice(base, 0, 1, 4);
  CHECK_THROWS_WITH(ops::add_(left, right, 1.0), "overlap");
  ops::add_(base, base, 1.0);
  CHECK(vals(base) == (V{2, 4, 6, 8}));
}
TEST(cpu_inplace_on_graph_tensors_needs_no_grad) {
  Tensor a = make({2}, {1, 2});
  a.requires_grad_(true);
  Tensor y = ops::mul_scalar(a, 2.0);
  CHECK_THROWS(ops::mul_(y, 2.0));          // a non-leaf with history
  NoGradGuard g;
  ops::mul_(a, 2.0);                        // a leaf under no_grad: the optimizer's way
  CHECK(vals(a) == (V{2, 4}));
}
TEST(cpu_unary_values) {
  Tensor x = make({4}, {-1, 0, 1, 4});
  CHECK(vals(ops::relu(x)) == (V{0, 0, 1, 4}));
  CHECK(vals(ops::neg(x)) == (V{1, -0.0, -1, -4}));
  CHECK_NEAR(vals(ops::sigmoid(x))[2], 1 / (1 + std::exp(-1.0)), 1e-6);
  CHECK_NEAR(vals(ops::tanh(x))[0], std::tanh(-1.0), 1e-6);
  CHECK_NEAR(vals(ops::exp(x))[3], std::exp(4.0), 1e-3);
  CHECK(vals(ops::sqrt(x))[3] == 2.0 && std::isnan(vals(ops::sqrt(x))[0]));
  CHECK(vals(ops::reciprocal(x))[3] == 0.25);
  CHECK(vals(ops::leaky_relu(x, 0.1))[0] == static_cast<double>(-0.1f));
  CHECK_NEAR(vals(ops::log(x))[3], std::log(4.0), 1e-6);
}
TEST(cpu_gelu_is_the_erf_form) {
  for (double v : {-3.0, -0.5, 0.0, 0.7, 2.5}) {
    const double want = 0.5 * v * (1 + std::erf(v / std::sqrt(2.0)));
    CHECK_NEAR(vals(ops::gelu(make({1}, {v})))[0], want, 1e-6);
  }
}
TEST(cpu_unary_on_strided_input_follows_logical_order) {
  Tensor a = make({2, 2}, {1, 2, 3, 4});
  CHECK(vals(ops::neg(ops::transpose(a, 0, 1))) == (V{-1, -3, -2, -4}));
}
TEST(cpu_sum_mean_over_every_dim) {
  Tensor a = make({2, 3}, {1, 2, 3, 4, 5, 6});
  CHECK(vals(ops::sum(a, std::nullopt, false)) == (V{21}));
  CHECK(vals(ops::sum(a, 0, false)) == (V{5, 7, 9}));
  CHECK(vals(ops::sum(a, -1, true)) == (V{6, 15}));
  CHECK(ops::sum(a, 1, true).shape() == (Shape{2, 1}));
  CHECK(vals(ops::mean(a, 1, false)) == (V{2, 5}));
  CHECK(ops::sum(a, std::nullopt, true).shape() == (Shape{1, 1}));
  CHECK_THROWS(ops::sum(a, 2, false));
  CHECK_THROWS(ops::sum(a, -3, false));
}
TEST(cpu_sum_all_accumulates_in_double) {
  Tensor a = Tensor::full({1 << 16}, 0.1, DType::F32, kCpu);
  CHECK_NEAR(vals(ops::sum(a, std::nullopt, false))[0], 6553.6, 0.01);
}
TEST(cpu_max_policy) {
  auto r = ops::max(make({4}, {1, 5, 5, 2}), std::nullopt, false);
  CHECK(vals(r.first) == (V{5}) && vals(r.second) == (V{1}));
  const double nan = std::numeric_limits<double>::quiet_NaN();
  auto n = ops::max(make({3}, {7, nan, nan}), std::nullopt, false);
  CHECK(std::isnan(vals(n.first)[0]) && vals(n.second) == (V{1}));
  CHECK(ops::argmax(make({2, 2}, {1, 9, 8, 3}), 1, false).dtype() == DType::I64);
  CHECK(vals(ops::argmax(make({2, 2}, {1, 9, 8, 3}), 0, false)) == (V{1, 0}));
}
TEST(cpu_reductions_reject_empty_input) {
  Tensor e = Tensor::zeros({0, 3}, DType::F32, kCpu);
  CHECK_THROWS(ops::sum(e, std::nullopt, false));
  CHECK_THROWS(ops::max(e, 0, false));
}
TEST(cpu_matmul_values_and_validation) {
  Tensor a = make({2, 3}, {1, 2, 3, 4, 5, 6}), b = make({3, 2}, {1, 0, 0, 1, 1, 1});
  CHECK(vals(ops::matmul(a, b)) == (V{4, 5, 10, 11}));
  CHECK_THROWS(ops::matmul(a, a));
  CHECK_THROWS(ops::matmul(make({3}, {1, 2, 3}), b));
  CHECK_THROWS_WITH(ops::matmul(a, make({3, 2}, {1, 0, 0, 1, 1, 1}, DType::F64)), "dtype mismatch");
}
TEST(cpu_batched_matmul_needs_equal_batches) {
  Tensor a = Tensor::full({2, 2, 3}, 1.0, DType::F32, kCpu), b = Tensor::full({2, 3, 4}, 2.0, DType::F32, kCpu);
  Tensor c = ops::matmul(a, b);
  CHECK(c.shape() == (Shape{2, 2, 4}) && vals(c)[0] == 6.0);
  CHECK_THROWS(ops::matmul(a, Tensor::full({3, 3, 4}, 2.0, DType::F32, kCpu)));
  CHECK_THROWS(ops::matmul(a, Tensor::full({3, 4}, 2.0, DType::F32, kCpu)));
}
TEST(cpu_matmul_reads_transposed_views) {
  Tensor a = make({2, 2}, {1, 2, 3, 4});
  CHECK(vals(ops::matmul(ops::transpose(a, 0, 1), a)) == (V{10, 14, 14, 20}));
  CHECK(vals(ops::gemm(a, true, a, false)) == (V{10, 14, 14, 20}));
  CHECK(vals(ops::gemm(a, false, a, true)) == (V{5, 11, 11, 25}));
}
TEST(cpu_matmul_with_an_empty_reduction_is_zero) {
  Tensor c = ops::matmul(Tensor::zeros({2, 0}, DType::F32, kCpu), Tensor::zeros({0, 3}, DType::F32, kCpu));
  CHECK(c.shape() == (Shape{2, 3}) && vals(c) == (V{0, 0, 0, 0, 0, 0}));
}
TEST(cpu_linear_bias_activation_and_residual) {
  Tensor x = make({1, 2}, {1, -1}), w = make({2, 2}, {1, 2, 3, 4}), b = make({2}, {0.5, 0.5});
  CHECK(vals(ops::linear(x, w, b, ops::Act::None, Tensor())) == (V{-1.5, -1.5}));
  CHECK(vals(ops::linear(x, w, b, ops::Act::Relu, Tensor())) == (V{0, 0}));
  CHECK(vals(ops::linear(x, w, Tensor(), ops::Act::None, make({1, 2}, {10, 20}))) == (V{8, 18}));
  CHECK(vals(ops::fused_linear_relu(make({1, 2}, {1, 1}), w, b)) == (V{4.5, 6.5}));
  CHECK_THROWS(ops::linear(x, make({3, 2}, {1, 2, 3, 4, 5, 6}), b, ops::Act::None, Tensor()));
  CHECK_THROWS(ops::linear(x, w, make({3}, {1, 2, 3}), ops::Act::None, Tensor()));
}
TEST(cpu_cast_goes_through_double_and_truncates_toward_zero) {
  Tensor f = make({4}, {-1.7, 0.2, 2.9, 300});
  CHECK(vals(ops::cast(f, DType::I32)) == (V{-1, 0, 2, 300}));
  CHECK(vals(ops::cast(f, DType::Bool)) == (V{1, 1, 1, 1}));
  CHECK(vals(ops::cast(make({2}, {0, -0.0}), DType::Bool)) == (V{0, 0}));
  Tensor same = ops::cast(f, DType::F32);
  CHECK(same.raw() == f.raw());
}
TEST(cpu_cast_of_an_integer_tensor_cuts_the_graph) {
  Tensor a = make({2}, {1.5, 2.5});
  a.requires_grad_(true);
  Tensor i = ops::cast(a, DType::I64);
  CHECK(!i.requires_grad() && i.is_leaf());
  Tensor h = ops::cast(a, DType::F64);
  CHECK(h.requires_grad() && !h.is_leaf());
}
TEST(cpu_to_always_copies) {
  Tensor a = make({2}, {1, 2});
  Tensor b = ops::to(a, kCpu);
  CHECK(!b.same_buffer(a) && vals(b) == vals(a));
  ops::fill_(b, 0.0);
  CHECK(vals(a) == (V{1, 2}));
}
TEST(cpu_contiguous_is_identity_on_packed_input) {
  Tensor a = make({2, 2}, {1, 2, 3, 4});
  CHECK(ops::contiguous(a).raw() == a.raw());
  Tensor t = ops::contiguous(ops::transpose(a, 0, 1));
  CHECK(t.is_contiguous() && !t.same_buffer(a) && vals(t) == (V{1, 3, 2, 4}));
}
TEST(cpu_flatten_and_reshape_with_inferred_extent) {
  Tensor a = Tensor::zeros({2, 3, 4}, DType::F32, kCpu);
  CHECK(ops::flatten(a, 1, 2).shape() == (Shape{2, 12}));
  CHECK(ops::flatten(a, 0, -1).shape() == (Shape{24}));
  CHECK(ops::reshape(a, {-1, 6}).shape() == (Shape{4, 6}));
  CHECK_THROWS(ops::reshape(a, {-1, -1}));
  CHECK_THROWS(ops::reshape(a, {5, -1}));
  CHECK_THROWS(ops::flatten(a, 2, 1));
}
TEST(cpu_softmax_rows_sum_to_one_and_are_shift_invariant) {
  Tensor a = make({2, 3}, {1, 2, 3, 1001, 1002, 1003});
  V s = vals(ops::softmax(a, 1));
  CHECK_NEAR(s[0] + s[1] + s[2], 1.0, 1e-6);
  CHECK_NEAR(s[0], s[3], 1e-6);
  V l = vals(ops::log_softmax(a, -1));
  CHECK_NEAR(std::exp(l[2]), s[2], 1e-6);
  CHECK_THROWS(ops::softmax(a, 2));
}
TEST(cpu_cross_entropy_and_nll_agree) {
  Tensor logits = make({2, 3}, {1, 2, 3, 3, 2, 1});
  Tensor targets = make({2}, {2, 0}, DType::I64);
  const double ce = vals(ops::cross_entropy(logits, targets))[0];
  const double nll = vals(ops::nll_loss(ops::log_softmax(logits, 1), targets, "mean"))[0];
  CHECK_NEAR(ce, nll, 1e-6);
  CHECK_NEAR(ce, -std::log(std::exp(3.0) / (std::exp(1.0) + std::exp(2.0) + std::exp(3.0))), 1e-6);
  CHECK(vals(ops::cross_entropy_host(logits, {2, 0}))[0] == ce);
  CHECK(ops::nll_loss(ops::log_softmax(logits, 1), targets, "none").shape() == (Shape{2}));
  CHECK_THROWS(ops::nll_loss(ops::log_softmax(logits, 1), targets, "median"));
}
TEST(cpu_class_targets_are_bounds_checked) {
  Tensor logits = make({1, 3}, {1, 2, 3});
  CHECK_THROWS(ops::cross_entropy(logits, make({1}, {3}, DType::I64)));
  CHECK_THROWS(ops::cross_entropy(logits, make({1}, {-1}, DType::I64)));
  CHECK_THROWS(ops::cross_entropy(logits, make({2}, {0, 1}, DType::I64)));
  CHECK_THROWS(ops::cross_entropy_host(logits, {5}));
}
TEST(cpu_embedding_gathers_rows_and_checks_indices) {
  Tensor w = make({3, 2}, {0, 1, 10, 11, 20, 21});
  CHECK(vals(ops::embedding(make({2, 2}, {2, 0, 1, 1}, DType::I64), w)) == (V{20, 21, 0, 1, 10, 11, 10, 11}));
  CHECK(ops::embedding(make({2, 2}, {2, 0, 1, 1}, DType::I32), w).shape() == (Shape{2, 2, 2}));
  CHECK_THROWS(ops::embedding(make({1}, {3}, DType::I64), w));
  CHECK_THROWS(ops::embedding(make({1}, {1}, DType::F32), w));
}
TEST(cpu_dropout_mask_is_a_pure_function_of_the_seed) {
  Tensor a = ops::dropout_mask({64}, 0.5, 1234, DType::F32, kCpu), b = ops::dropout_mask({64}, 0.5, 1234, DType::F32, kCpu);
  CHECK(vals(a) == vals(b));
  CHECK(vals(a) != vals(ops::dropout_mask({64}, 0.5, 1235, DType::F32, kCpu)));
  for (double v : vals(a)) CHECK(v == 0.0 || v == 2.0);
  CHECK(vals(ops::dropout_mask({8}, 0.0, 1, DType::F32, kCpu)) == V(8, 1.0));
  CHECK_THROWS(ops::dropout_mask({8}, 1.0, 1, DType::F32, kCpu));
  CHECK_THROWS(ops::dropout_mask({8}, -0.1, 1, DType::F32, kCpu));
}
TEST(cpu_conv_and_pool_geometry_is_validated) {
  Tensor x = Tensor::zeros({1, 2, 5, 5}, DType::F32, kCpu), w = Tensor::zeros({3, 2, 3, 3}, DType::F32, kCpu), b = Tensor::zeros({3}, DType::F32, kCpu);
  CHECK(ops::conv2d(x, w, b, 1, 1, 1, 1).shape() == (Shape{1, 3, 5, 5}));
  CHECK(ops::conv2d(x, w, b, 2, 2, 0, 0).shape() == (Shape{1, 3, 2, 2}));
  CHECK_THROWS(ops::conv2d(x, Tensor::zeros({3, 4, 3, 3}, DType::F32, kCpu), b, 1, 1, 0, 0));  // channel mismatch
  CHECK_THROWS(ops::conv2d(x, w, b, 0, 1, 0, 0));                                              // zero stride
  CHECK_THROWS(ops::conv2d(x, Tensor::zeros({3, 2, 7, 7}, DType::F32, kCpu), b, 1, 1, 0, 0));  // kernel larger than the input
  CHECK(ops::maxpool2d(x, 2, 2, 2, 2, 0, 0).shape() == (Shape{1, 2, 2, 2}));
  CHECK_THROWS(ops::maxpool2d(x, 2, 2, 2, 2, 2, 2));                                           // padding above half the window
}
TEST(cpu_layer_norm_normalises_the_last_dimension) {
  Tensor x = make({2, 4}, {1, 2, 3, 4, 2, 4, 6, 8});
  V y = vals(ops::layer_norm(x, Tensor(), Tensor(), 0.0));
  CHECK_NEAR(y[0] + y[1] + y[2] + y[3], 0.0, 1e-6);
  CHECK_NEAR(y[0], y[4], 1e-6);  // scale invariance
  V z = vals(ops::layer_norm(x, make({4}, {2, 2, 2, 2}), make({4}, {1, 1, 1, 1}), 1e-5));
  CHECK_NEAR(z[3], 2 * y[3] + 1, 1e-4);
}
TEST(cpu_isfinite_all) {
  CHECK(ops::isfinite_all(make({2}, {1, 2})));
  CHECK(!ops::isfinite_all(make({2}, {1, std::numeric_limits<double>::infinity()})));
  CHECK(!ops::isfinite_all(make({2}, {std::numeric_limits<double>::quiet_NaN(), 0})));
  CHECK(ops::isfinite_all(make({2}, {1, 2}, DType::I64)));
  CHECK(ops::isfinite_all(Tensor::zeros({0}, DType::F32, kCpu)));
}
TEST(cpu_amp_unscale_reports_whether_every_value_is_finite) {
  auto ok = ops::amp_unscale_to_f32_and_check(make({2}, {2, 4}), 0.5);
  CHECK(ok.second && vals(ok.first) == (V{1, 2}) && ok.first.dtype() == DType::F32);
  auto bad = ops::amp_unscale_to_f32_and_check(make({2}, {2, std::numeric_limits<double>::infinity()}), 0.5);
  CHECK(!bad.second);
  CHECK(ops::amp_unscale_to_f32_and_check(Tensor::zeros({0}, DType::F32, kCpu), 0.5).second);
}
TEST(cpu_copy_range_and_scalar_access_are_bounds_checked) {
  Tensor a = make({4}, {1, 2, 3, 4}), b = Tensor::zeros({4}, DType::F32, kCpu);
  ops::copy_range(b, 1, a, 0, 3);
  CHECK(vals(b) == (V{0, 1, 2, 3}));
  CHECK_THROWS(ops::copy_range(b, 2, a, 0, 3));
  CHECK_THROWS(ops::copy_range(b, 0, a, 2, 3));
  CHECK_THROWS(ops::read_scalar(a, 4));
  CHECK_THROWS(ops::write_scalar(a, -1, 0.0));
}
TEST(cpu_unbroadcast_sums_back_to_the_source_shape) {
  Tensor g = make({2, 3}, {1, 2, 3, 4, 5, 6});
  CHECK(vals(ops::unbroadcast(g, {3})) == (V{5, 7, 9}));
  CHECK(vals(ops::unbroadcast(g, {2, 1})) == (V{6, 15}));
  CHECK(vals(ops::unbroadcast(g, {1})) == (V{21}));
  CHECK(ops::unbroadcast(g, {2, 3}).raw() == g.raw());
}

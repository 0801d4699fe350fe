// Tensor / Buffer aliasing, semantic operators on the CPU backend and the autograd engine.
// (reference project: tests/cpp operators and autograd domains; src/autograd/engine.cpp:78-206)
#include <cmath>
#include <vector>

#include "check.h"
#include "ob/ops.h"
#include "ob/tensor.h"

using namespace ob;

namespace {
const Device kCpu;

Tensor vec(std::initializer_list<double> values, bool grad = false, DType dt = DType::F32) {
  Tensor t = Tensor::empty({static_cast<int64_t>(values.size())}, dt, kCpu);
  int64_t i = 0;
  for (double v : values) ops::write_scalar(t, i++, v);
  if (grad) t.requires_grad_(true);
  return t;
}
Tensor mat(int64_t r, int64_t c, std::initializer_list<double> values, bool grad = false) {
  Tensor t = Tensor::empty({r, c}, DType::F32, kCpu);
  int64_t i = 0;
  for (double v : values) ops::write_scalar(t, i++, v);
  if (grad) t.requires_grad_(true);
  return t;
}
std::vector<double> values(const Tensor& t) {
  Tensor c = ops::contiguous(t);
  std::vector<double> out;
  for (int64_t i = 0; i < c.numel(); ++i) out.push_back(ops::read_scalar(c, i));
  return out;
}
}  // namespace

TEST(views_share_one_buffer_and_its_version) {
  Tensor base = mat(2, 3, {0, 1, 2, 3, 4, 5});
  Tensor row = ops::index(base, 1);
  Tensor tr = ops::transpose(base, 0, 1);
  CHECK(row.same_buffer(base) && tr.same_buffer(base));
  CHECK_EQ(row.offset(), 3);
  CHECK(tr.shape() == (Shape{3, 2}) && tr.strides() == (Shape{1, 3}));
  CHECK(!tr.is_contiguous());
  const uint64_t v0 = base.version();
  ops::fill_(row, 9.0);  // one logical write, one bump, visible through every alias
  CHECK_EQ(base.version(), v0 + 1);
  CHECK_EQ(tr.version(), v0 + 1);
  CHECK(values(base) == (std::vector<double>{0, 1, 2, 9, 9, 9}));
  ops::fill_(row, 9.0);  // same value still counts as a write
  CHECK_EQ(base.version(), v0 + 2);
  Tensor r2 = ops::reshape(base, {3, 2});  // metadata only
  CHECK(r2.same_buffer(base));
  CHECK_EQ(base.version(), v0 + 2);
  CHECK_THROWS(ops::reshape(tr, {6}));     // a view needs packed storage
  CHECK_THROWS(ops::reshape(base, {4, 2}));
}

TEST(slice_and_index_bounds) {
  Tensor a = vec({0, 1, 2, 3, 4, 5});
  CHECK(values(ops::slice(a, 0, 2, 5)) == (std::vector<double>{2, 3, 4}));
  CHECK(values(ops::slice(a, 0, 4, 4)).empty());
  CHECK_THROWS(ops::slice(a, 0, 3, 7));
  CHECK_THROWS(ops::slice(a, 1, 0, 1));
  CHECK_THROWS(ops::index(a, 6));
  CHECK(values(ops::index(a, -1)) == (std::vector<double>{5}));
}

TEST(elementwise_broadcast_and_composites) {
  Tensor a = mat(2, 3, {1, 2, 3, 4, 5, 6});
  Tensor row = vec({10, 20, 30});
  CHECK(values(ops::add(a, row)) == (std::vector<double>{11, 22, 33, 14, 25, 36}));
  CHECK(values(ops::mul(a, ops::reshape(vec({2, 3}), {2, 1}))) == (std::vector<double>{2, 4, 6, 12, 15, 18}));
  CHECK(values(ops::sub(a, row)) == (std::vector<double>{-9, -18, -27, -6, -15, -24}));
  const std::vector<double> q = values(ops::div(row, vec({2, 4, 5})));
  CHECK_NEAR(q[0], 5.0, 1e-6); CHECK_NEAR(q[1], 5.0, 1e-6); CHECK_NEAR(q[2], 6.0, 1e-6);
  CHECK_THROWS(ops::add(a, vec({1, 2})));
  CHECK_THROWS(ops::add(a, vec({1, 2, 3}, false, DType::F64)));  // no implicit promotion
  CHECK(values(ops::add_scalar(row, 0.5)) == (std::vector<double>{10.5, 20.5, 30.5}));
  CHECK(values(ops::mul_scalar(row, -1.0)) == (std::vector<double>{-10, -20, -30}));
}

TEST(inplace_add_rejects_partial_overlap) {
  Tensor a = vec({0, 1, 2, 3, 4, 5, 6, 7});
  Tensor lo = ops::slice(a, 0, 0, 6), hi = ops::slice(a, 0, 2, 8);
  CHECK_THROWS_WITH(ops::add_(lo, hi, 1.0), "overlap");
  const uint64_t v0 = a.version();
  ops::add_(a, a, 1.0);  // identical ranges are fine
  CHECK_EQ(a.version(), v0 + 1);
  CHECK(values(a)[7] == 14.0);
  ops::mul_(a, 0.5);
  CHECK(values(a)[7] == 7.0);
}

TEST(reductions_and_extrema_policy) {
  Tensor a = mat(2, 3, {1, 5, 5, -2, -7, 0});
  CHECK(values(ops::sum(a, std::nullopt, false)) == (std::vector<double>{2}));
  CHECK(values(ops::sum(a, 0, false)) == (std::vector<double>{-1, -2, 5}));
  CHECK(ops::sum(a, 1, true).shape() == (Shape{2, 1}));
  CHECK_NEAR(values(ops::mean(a, -1, false))[0], 11.0 / 3.0, 1e-6);
  CHECK_NEAR(values(ops::mean(a, -1, false))[1], -3.0, 1e-6);
  auto [vals, idx] = ops::max(a, 1, false);
  CHECK(values(vals) == (std::vector<double>{5, 0}));
  CHECK(values(idx) == (std::vector<double>{1, 2}));  // the first maximum wins
  CHECK(idx.dtype() == DType::I64);
  Tensor with_nan = vec({1, NAN, 3, NAN});
  CHECK(values(ops::argmax(with_nan, std::nullopt, false)) == (std::vector<double>{1}));  // first NaN wins
  CHECK_THROWS(ops::sum(Tensor::zeros({0}, DType::F32, kCpu), std::nullopt, false));
  CHECK_THROWS(ops::sum(a, 2, false));
}

TEST(matmul_shapes_and_values) {
  Tensor a = mat(2, 3, {1, 2, 3, 4, 5, 6}), b = mat(3, 2, {1, 0, 0, 1, 1, 1});
  CHECK(values(ops::matmul(a, b)) == (std::vector<double>{4, 5, 10, 11}));
  CHECK(values(ops::gemm(a, true, a, false)).size() == 9u);
  CHECK_THROWS(ops::matmul(a, a));
  CHECK_THROWS(ops::matmul(vec({1, 2, 3}), b));  // rank 1 is not a matrix
  Tensor batch_a = Tensor::full({2, 2, 3}, 1.0, DType::F32, kCpu), batch_b = Tensor::full({2, 3, 4}, 2.0, DType::F32, kCpu);
  Tensor c = ops::matmul(batch_a, batch_b);
  CHECK(c.shape() == (Shape{2, 2, 4}));
  CHECK(values(c)[5] == 6.0);
  CHECK_THROWS(ops::matmul(batch_a, Tensor::full({3, 3, 4}, 2.0, DType::F32, kCpu)));  // batch extents must match
}

TEST(softmax_cross_entropy_and_nll) {
  Tensor logits = mat(2, 3, {1, 2, 3, 1, 1, 1});
  const std::vector<double> p = values(ops::softmax(logits, 1));
  CHECK_NEAR(p[0] + p[1] + p[2], 1.0, 1e-6);
  CHECK_NEAR(p[3], 1.0 / 3.0, 1e-6);
  const std::vector<double> lp = values(ops::log_softmax(logits, 1));
  CHECK_NEAR(lp[2], std::log(p[2]), 1e-6);
  Tensor loss = ops::cross_entropy_host(logits, {2, 0});
  CHECK(loss.shape() == (Shape{1}));
  CHECK_NEAR(values(loss)[0], -(std::log(p[2]) + std::log(1.0 / 3.0)) / 2.0, 1e-6);
  CHECK_THROWS(ops::cross_entropy_host(logits, {3, 0}));  // target out of range
  CHECK_THROWS(ops::cross_entropy_host(logits, {1}));     // one target per row
  Tensor targets = Tensor::zeros({2}, DType::I64, kCpu);
  ops::write_scalar(targets, 0, 2);
  CHECK_NEAR(values(ops::nll_loss(ops::log_softmax(logits, 1), targets, "mean"))[0], values(loss)[0], 1e-6);
  CHECK(ops::nll_loss(ops::log_softmax(logits, 1), targets, "none").shape() == (Shape{2}));
  CHECK_THROWS(ops::nll_loss(ops::log_softmax(logits, 1), targets, "median"));
}

TEST(backward_accumulates_into_leaves_and_seeds_with_ones) {
  Tensor x = vec({1, 2, 3}, true), w = vec({4, 5, 6}, true);
  Tensor y = ops::sum(ops::mul(x, w), std::nullopt, false);
  CHECK(!y.is_leaf() && y.requires_grad());
  y.backward();
  CHECK(values(x.grad()) == (std::vector<double>{4, 5, 6}));
  CHECK(values(w.grad()) == (std::vector<double>{1, 2, 3}));
  // A second graph accumulates into the existing gradient, which keeps its own storage.
  Tensor g_before = x.grad();
  ops::sum(ops::mul_scalar(x, 2.0), std::nullopt, false).backward();
  CHECK(values(x.grad()) == (std::vector<double>{6, 7, 8}));
  CHECK(!x.grad().same_buffer(w.grad()));
  x.zero_grad();
  CHECK(!x.grad().defined());
  (void)g_before;
}

TEST(a_tensor_used_twice_receives_both_contributions) {
  Tensor x = vec({2, 3}, true);
  Tensor y = ops::sum(ops::add(ops::mul(x, x), x), std::nullopt, false);  // x^2 + x
  y.backward();
  CHECK(values(x.grad()) == (std::vector<double>{5, 7}));
}

TEST(released_graph_and_retain_graph) {
  Tensor x = vec({1, 2}, true);
  Tensor y = ops::sum(ops::mul(x, x), std::nullopt, false);
  y.backward(true);
  y.backward(false);  // retained once: a second pass is allowed and accumulates
  CHECK(values(x.grad()) == (std::vector<double>{4, 8}));
  CHECK_THROWS_WITH(y.backward(), "freed");  // history was released by the previous pass
}

TEST(saved_tensor_modified_in_place_is_detected) {
  Tensor x = vec({1, 2}, true), w = vec({3, 4});
  Tensor y = ops::sum(ops::mul(x, w), std::nullopt, false);  // the product saves w
  ops::fill_(w, 0.0);
  CHECK_THROWS_WITH(y.backward(), "modified in-place");
}

TEST(no_grad_records_nothing_and_restores_the_mode) {
  Tensor x = vec({1, 2}, true);
  CHECK(grad_enabled());
  {
    NoGradGuard guard;
    CHECK(!grad_enabled());
    Tensor y = ops::mul(x, x);
    CHECK(y.is_leaf() && !y.requires_grad());
  }
  CHECK(grad_enabled());
  Tensor d = x.detach();
  CHECK(d.same_buffer(x) && !d.requires_grad());
}

TEST(backward_needs_a_graph_and_validates_hand_set_gradients) {
  Tensor plain = vec({1, 2});
  CHECK_THROWS(ops::sum(plain, std::nullopt, false).backward());
  Tensor x = vec({1, 2}, true);
  CHECK_THROWS(x.set_grad(vec({1, 2, 3})));                      // shape
  CHECK_THROWS(x.set_grad(vec({1, 2}, false, DType::F64)));      // dtype
  x.set_grad(vec({7, 8}));
  ops::sum(x, std::nullopt, false).backward();
  CHECK(values(x.grad()) == (std::vector<double>{8, 9}));
}

TEST(hooks_and_finalizers_run_once_per_backward) {
  Tensor x = vec({1, 2}, true);
  int hook_runs = 0, finalizer_runs = 0;
  x.impl()->ag().post_accumulate_hooks.push_back([&] { ++hook_runs; });
  Tensor y = ops::sum(ops::mul(x, x), std::nullopt, false);
  // Finalizers of a produced tensor live on its node, those of a leaf on the leaf itself.
  y.grad_fn()->finalizers.emplace_back(42, [&] { ++finalizer_runs; });
  x.impl()->ag().finalizers.emplace_back(42, [&] { ++finalizer_runs; });  // same key: one run
  y.backward();
  CHECK_EQ(hook_runs, 1);
  CHECK_EQ(finalizer_runs, 1);
}

TEST(float64_graph_keeps_its_dtype) {
  Tensor x = vec({0.5, 1.5}, true, DType::F64);
  Tensor y = ops::sum(ops::exp(x), std::nullopt, false);
  y.backward();
  CHECK(x.grad().dtype() == DType::F64);
  CHECK_NEAR(values(x.grad())[1], std::exp(1.5), 1e-12);
}

TEST(cast_and_transfer_contracts_on_the_cpu) {
  Tensor x = vec({1.25, -2.5}, true);
  Tensor d = ops::cast(x, DType::F64);
  CHECK(d.dtype() == DType::F64 && d.requires_grad());
  ops::sum(d, std::nullopt, false).backward();
  CHECK(x.grad().dtype() == DType::F32);
  CHECK(values(x.grad()) == (std::vector<double>{1, 1}));
  Tensor same = ops::to(x, kCpu);
  CHECK(same.device() == kCpu);
  Tensor h = ops::cast(vec({1.0, 65504.0}), DType::F16);
  CHECK(values(ops::cast(h, DType::F32)) == (std::vector<double>{1.0, 65504.0}));
}

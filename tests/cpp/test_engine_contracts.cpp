// Autograd engine contracts through the C++ API: seeds, accumulation, released graphs, hooks and
// finalizers, version checks, deep chains, gradient destinations.
// (reference project: tests/cpp/test_autograd_engine.cpp, src/autograd/engine.cpp:78-206)
#include <vector>

#include "check.h"
#include "ob/ops.h"
#include "ob/tensor.h"

using namespace ob;

namespace {
const Device kCpu;
Tensor leaf(std::initializer_list<double> v) {
  Tensor t = Tensor::empty({static_cast<int64_t>(v.size())}, DType::F32, kCpu);
  int64_t i = 0;
  for (double x : v) ops::write_scalar(t, i++, x);
  t.requires_grad_(true);
  return t;
}
std::vector<double> vals(const Tensor& t) {
  std::vector<double> out;
  Tensor c = ops::contiguous(t);
  for (int64_t i = 0; i < c.numel(); ++i) out.push_back(ops::read_scalar(c, i));
  return out;
}
using V = std::vector<double>;
}  // namespace

TEST(engine_seed_is_ones_for_non_scalar_roots) {
  Tensor x = leaf({1, 2, 3});
  ops::mul_scalar(x, 3.0).backward();
  CHECK(vals(x.grad()) == (V{3, 3, 3}));
}
TEST(engine_root_must_require_grad) {
  Tensor c = Tensor::full({2}, 1.0, DType::F32, kCpu);
  CHECK_THROWS_WITH(c.backward(), "does not require grad");
}
TEST(engine_leaf_root_receives_the_seed) {
  Tensor x = leaf({1, 2});
  x.backward();
  CHECK(vals(x.grad()) == (V{1, 1}));
}
TEST(engine_gradients_accumulate_until_zero_grad) {
  Tensor x = leaf({1, 2});
  ops::sum(ops::mul(x, x), std::nullopt, false).backward();
  ops::sum(x, std::nullopt, false).backward();
  CHECK(vals(x.grad()) == (V{3, 5}));
  x.zero_grad();
  CHECK(!x.grad().defined());
}
TEST(engine_grad_is_an_independent_graph_free_leaf) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::mul_scalar(x, 2.0);
  y.backward();
  Tensor g = x.grad();
  CHECK(g.is_leaf() && !g.requires_grad() && !g.same_buffer(y) && !g.same_buffer(x));
  CHECK(g.dtype() == x.dtype() && g.device() == x.device() && g.shape() == x.shape());
}
TEST(engine_second_backward_on_a_released_graph_names_the_remedy) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::sum(ops::mul(x, x), std::nullopt, false);
  y.backward();
  CHECK_THROWS_WITH(y.backward(), "Cannot call backward twice on a freed graph. Use retain_graph=True.");
  CHECK(vals(x.grad()) == (V{2, 4}));  // the failed call committed nothing
}
TEST(engine_retain_graph_allows_repeated_backward) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::sum(ops::mul(x, x), std::nullopt, false);
  y.backward(true);
  y.backward(true);
  y.backward(false);
  CHECK(vals(x.grad()) == (V{6, 12}));
  CHECK_THROWS(y.backward());
}
TEST(engine_shared_subgraph_is_evaluated_once_per_backward) {
  Tensor x = leaf({2});
  Tensor h = ops::mul(x, x);            // used twice below
  ops::add(h, h).backward();
  CHECK(vals(x.grad()) == (V{8}));      // d(2 x^2)/dx = 4x
}
TEST(engine_diamond_accumulates_both_paths) {
  Tensor x = leaf({3});
  ops::mul(ops::add_scalar(x, 1.0), ops::mul_scalar(x, 2.0)).backward();   // (x+1) * 2x -> 4x + 2
  CHECK(vals(x.grad()) == (V{14}));
}
TEST(engine_no_grad_builds_no_graph) {
  Tensor x = leaf({1});
  {
    NoGradGuard g;
    CHECK(!grad_enabled());
    Tensor y = ops::mul_scalar(x, 2.0);
    CHECK(y.is_leaf() && !y.requires_grad());
    {
      NoGradGuard inner;
      CHECK(!grad_enabled());
    }
    CHECK(!grad_enabled());
  }
  CHECK(grad_enabled());
}
TEST(engine_detach_shares_storage_without_history) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::mul_scalar(x, 2.0);
  Tensor d = y.detach();
  CHECK(d.same_buffer(y) && d.is_leaf() && !d.requires_grad());
  Tensor plain = Tensor::zeros({1}, DType::F32, kCpu);
  CHECK(plain.detach().raw() == plain.raw());
}
TEST(engine_saved_tensor_modified_in_place_is_detected_at_preflight) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::sum(ops::mul(x, x), std::nullopt, false);
  {
    NoGradGuard g;
    ops::fill_(x, 5.0);
  }
  CHECK_THROWS_WITH(y.backward(), "was modified in-place after it was saved for backward (expected version");
  CHECK(!x.grad().defined());
}
TEST(engine_writes_to_unsaved_tensors_do_not_invalidate) {
  Tensor x = leaf({1, 2});
  Tensor y = ops::sum(ops::add_scalar(x, 1.0), std::nullopt, false);   // add saves nothing
  {
    NoGradGuard g;
    ops::fill_(x, 5.0);
  }
  y.backward();
  CHECK(vals(x.grad()) == (V{1, 1}));
}
TEST(engine_hooks_run_once_per_contributing_leaf_after_the_commit) {
  Tensor a = leaf({1}), b = leaf({2}), unused = leaf({3});
  int hits_a = 0, hits_b = 0, hits_unused = 0;
  bool grad_visible = false;
  a.impl()->ag().post_accumulate_hooks.push_back([&] { ++hits_a; grad_visible = a.grad().defined() && b.grad().defined(); });
  b.impl()->ag().post_accumulate_hooks.push_back([&] { ++hits_b; });
  unused.impl()->ag().post_accumulate_hooks.push_back([&] { ++hits_unused; });
  ops::add(ops::mul(a, b), a).backward();   // a is reached through two paths
  CHECK_EQ(hits_a, 1);
  CHECK_EQ(hits_b, 1);
  CHECK_EQ(hits_unused, 0);
  CHECK(grad_visible);                      // every leaf was committed before the first hook ran
}
TEST(engine_finalizers_run_once_per_key_after_hooks) {
  Tensor a = leaf({1}), b = leaf({2});
  std::vector<int> order;
  a.impl()->ag().post_accumulate_hooks.push_back([&] { order.push_back(1); });
  a.impl()->ag().finalizers.emplace_back(7, [&] { order.push_back(2); });
  b.impl()->ag().finalizers.emplace_back(7, [&] { order.push_back(2); });   // same key: runs once
  b.impl()->ag().finalizers.emplace_back(8, [&] { order.push_back(3); });
  ops::mul(a, b).backward();
  CHECK(order == (std::vector<int>{1, 2, 3}));
}
TEST(engine_failure_inside_a_formula_commits_nothing) {
  struct Exploding : Node {
    const char* name() const override { return "ExplodingNode"; }
    std::vector<Tensor> backward(const Tensor&) override { throw std::runtime_error("formula failed"); }
  };
  Tensor a = leaf({1}), b = leaf({2});
  Tensor bad = Tensor::zeros({1}, DType::F32, kCpu);
  auto node = std::make_shared<Exploding>();
  node->set_inputs({b});
  node->out_shape = bad.shape(); node->out_dtype = bad.dtype(); node->out_device = bad.device();
  bad.requires_grad_(true);
  bad.impl()->ag().grad_fn = node;
  bad.impl()->ag().history = History::Live;
  CHECK_THROWS_WITH(ops::add(ops::mul_scalar(a, 2.0), bad).backward(), "formula failed");
  CHECK(!a.grad().defined() && !b.grad().defined());
}
TEST(engine_gradient_shape_is_validated) {
  struct WrongShape : Node {
    const char* name() const override { return "WrongShapeNode"; }
    std::vector<Tensor> backward(const Tensor&) override { return {Tensor::zeros({3}, DType::F32, Device())}; }
  };
  Tensor a = leaf({1, 2});
  Tensor out = Tensor::zeros({2}, DType::F32, kCpu);
  auto node = std::make_shared<WrongShape>();
  node->set_inputs({a});
  node->out_shape = out.shape(); node->out_dtype = out.dtype(); node->out_device = out.device();
  out.requires_grad_(true);
  out.impl()->ag().grad_fn = node;
  out.impl()->ag().history = History::Live;
  CHECK_THROWS_WITH(out.backward(), "WrongShapeNode");
  CHECK(!a.grad().defined());
}
TEST(engine_addend_offer_replaces_the_running_sum_when_taken) {
  // y = h + f(h) with h = 3 * x: the skip path delivers its gradient to h's producer first; f is then
  // offered that running sum.  A formula that takes the offer returns (own + addend) and the engine
  // must not add the addend a second time; one that ignores it is accumulated as before.
  struct Branch : Node {
    bool take = false;
    int offers = 0;
    const char* name() const override { return "BranchNode"; }
    std::vector<Tensor> backward(const Tensor& g) override {
      Tensor own = ops::mul_scalar(g, 10.0);
      Tensor addend = offered_addend(0);
      if (addend.defined()) ++offers;
      if (take && addend.defined()) {
        take_addend(0);
        return {ops::add(own, addend)};
      }
      return {own};
    }
  };
  for (bool take : {false, true}) {
    Tensor x = leaf({1, 2});
    Tensor h = ops::mul_scalar(x, 3.0);
    Tensor out = Tensor::zeros({2}, DType::F32, kCpu);
    auto node = std::make_shared<Branch>();
    node->take = take;
    node->set_inputs({h});
    node->out_shape = out.shape(); node->out_dtype = out.dtype(); node->out_device = out.device();
    out.requires_grad_(true);
    out.impl()->ag().grad_fn = node;
    out.impl()->ag().history = History::Live;
    ops::add(h, out).backward();
    CHECK(node->offers == 1);
    CHECK(vals(x.grad()) == (V{33, 33}));   // 3 * (1 + 10) either way
    CHECK(node->grad_addend.empty() && node->addend_taken.empty());
  }
}
TEST(engine_addend_is_not_offered_to_a_node_that_reaches_the_producer_twice) {
  struct Twice : Node {
    int offers = 0;
    const char* name() const override { return "TwiceNode"; }
    std::vector<Tensor> backward(const Tensor& g) override {
      if (offered_addend(0).defined() || offered_addend(1).defined()) ++offers;
      return {g, g};
    }
  };
  Tensor x = leaf({1});
  Tensor h = ops::mul_scalar(x, 2.0);
  Tensor out = Tensor::zeros({1}, DType::F32, kCpu);
  auto node = std::make_shared<Twice>();
  node->set_inputs({h, h});
  node->out_shape = out.shape(); node->out_dtype = out.dtype(); node->out_device = out.device();
  out.requires_grad_(true);
  out.impl()->ag().grad_fn = node;
  out.impl()->ag().history = History::Live;
  ops::add(h, out).backward();
  CHECK(node->offers == 0);
  CHECK(vals(x.grad()) == (V{6}));
}
TEST(engine_deep_chains_do_not_recurse) {
  Tensor x = leaf({1});
  Tensor y = x;
  for (int i = 0; i < 6000; ++i) y = ops::add_scalar(y, 0.0);
  y.backward();
  CHECK(vals(x.grad()) == (V{1}));
}
TEST(engine_wide_fan_in_accumulates_in_order) {
  Tensor x = leaf({1});
  Tensor total = ops::mul_scalar(x, 1.0);
  for (int i = 2; i <= 50; ++i) total = ops::add(total, ops::mul_scalar(x, static_cast<double>(i)));
  total.backward();
  CHECK(vals(x.grad()) == (V{1275}));
}
TEST(engine_preassigned_slot_receives_the_weight_gradient_in_place) {
  // A leaf with a gradient slot and one consumer: the formula is offered the slot and writes it directly.
  Tensor x = Tensor::full({4, 3}, 1.0, DType::F32, kCpu);
  Tensor w = Tensor::full({3, 2}, 0.5, DType::F32, kCpu);
  w.requires_grad_(true);
  Tensor slot = Tensor::zeros({3, 2}, DType::F32, kCpu);
  w.impl()->ag().grad_slot = slot.impl();
  int hooks = 0;
  w.impl()->ag().post_accumulate_hooks.push_back([&] { ++hooks; });
  const uint64_t v0 = slot.version();
  ops::sum(ops::matmul(x, w), std::nullopt, false).backward();
  CHECK(w.grad().same_buffer(slot) && w.grad().data() == slot.data());
  CHECK(vals(slot) == V(6, 4.0));
  CHECK(slot.version() > v0);
  CHECK_EQ(hooks, 1);
  // A second backward accumulates into the slot instead of overwriting it.
  ops::sum(ops::matmul(x, w), std::nullopt, false).backward();
  CHECK(vals(slot) == V(6, 8.0));
  CHECK_EQ(hooks, 2);
}
TEST(engine_slot_with_two_consumers_is_filled_after_the_last_one) {
  Tensor w = leaf({1, 2});
  Tensor slot = Tensor::zeros({2}, DType::F32, kCpu);
  w.impl()->ag().grad_slot = slot.impl();
  ops::sum(ops::add(ops::mul_scalar(w, 2.0), ops::mul_scalar(w, 3.0)), std::nullopt, false).backward();
  CHECK(vals(slot) == (V{5, 5}) && w.grad().same_buffer(slot));
}
TEST(engine_zero_grad_then_backward_overwrites_the_slot) {
  Tensor w = leaf({1, 2});
  Tensor slot = Tensor::full({2}, 99.0, DType::F32, kCpu);
  w.impl()->ag().grad_slot = slot.impl();
  ops::sum(ops::mul_scalar(w, 2.0), std::nullopt, false).backward();
  CHECK(vals(slot) == (V{2, 2}));       // stale contents are not accumulated into
  w.zero_grad();
  ops::sum(ops::mul_scalar(w, 7.0), std::nullopt, false).backward();
  CHECK(vals(slot) == (V{7, 7}));
}

// KernelRegistry rules and Dispatcher selection.
// (reference project: tests/cpp dispatcher cases; src/dispatch/kernel_registry.cpp:37-88,
// src/dispatch/dispatcher.cpp:43-122)
#include "check.h"
#include "ob/dispatch.h"
#include "ob/ops.h"

using namespace ob;

namespace {
int g_calls = 0;
void kernel_a(OpCall&) { g_calls += 1; }
void kernel_b(OpCall&) { g_calls += 100; }

KernelRegistry small_registry() {
  KernelRegistry r;
  r.add_schema(Schema{OperatorId::Add, "add", 2, false});
  r.add_schema(Schema{OperatorId::Sub, "sub", 2, true});
  return r;
}
}  // namespace

TEST(registry_rejects_duplicates_and_kernels_on_composites) {
  KernelRegistry r = small_registry();
  CHECK_THROWS(r.add_schema(Schema{OperatorId::Add, "add_again", 2, false}));  // same id
  CHECK_THROWS(r.add_schema(Schema{OperatorId::Mul, "add", 2, false}));        // same name
  r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kContiguous, Capability::None}, kernel_a, "a");
  CHECK_THROWS(r.add_kernel(OperatorId::Sub, Constraints{Backend::CPU, kMaskF32, kContiguous, Capability::None}, kernel_a, "sub"));
  CHECK_THROWS(r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kContiguous, Capability::None}, nullptr, "null"));
  // Overlap: same backend, an intersecting dtype mask and an intersecting layout mask.
  CHECK_THROWS(r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32 | kMaskF64, kContiguous | kStrided, Capability::None}, kernel_b, "b"));
  // Disjoint layout: allowed.
  r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kStrided, Capability::None}, kernel_b, "b_strided");
  CHECK_THROWS(r.add_kernel(OperatorId::Mul, Constraints{Backend::CPU, kMaskF32, kContiguous, Capability::None}, kernel_a, "no schema"));
}

TEST(registry_freeze_turns_missing_builtins_into_errors) {
  KernelRegistry r = small_registry();
  r.expect_kernel(OperatorId::Add, Backend::CPU, DType::F32);
  CHECK_THROWS_WITH(r.freeze(), "built-in kernel missing");
  KernelRegistry ok = small_registry();
  ok.expect_kernel(OperatorId::Add, Backend::CPU, DType::F32);
  ok.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kContiguous, Capability::None}, kernel_a, "a");
  CHECK_THROWS(ok.find(OperatorId::Add, Backend::CPU, DType::F32, kContiguous));  // lookup needs a frozen registry
  ok.freeze();
  CHECK(ok.frozen());
  CHECK_THROWS_WITH(ok.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF64, kContiguous, Capability::None}, kernel_b, "late"), "frozen");
  CHECK(ok.find(OperatorId::Add, Backend::CPU, DType::F32, kContiguous) != nullptr);
  CHECK(ok.find(OperatorId::Add, Backend::CPU, DType::F64, kContiguous) == nullptr);
  CHECK(ok.find(OperatorId::Add, Backend::CUDA, DType::F32, kContiguous) == nullptr);
}

TEST(dispatcher_selects_by_dtype_then_layout_and_reports_both) {
  KernelRegistry r = small_registry();
  r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kContiguous | kEmpty, Capability::None}, kernel_a, "packed");
  r.add_kernel(OperatorId::Add, Constraints{Backend::CPU, kMaskF32, kStrided, Capability::None}, kernel_b, "strided");
  r.freeze();
  Dispatcher d(std::move(r));
  const Device cpu;
  CHECK_EQ(std::string(d.select(DispatchRequest{OperatorId::Add, cpu, DType::F32, kContiguous}).name), std::string("packed"));
  CHECK_EQ(std::string(d.select(DispatchRequest{OperatorId::Add, cpu, DType::F32, kStrided}).name), std::string("strided"));
  CHECK_THROWS_WITH(d.select(DispatchRequest{OperatorId::Add, cpu, DType::F64, kContiguous}), "unsupported dtype float64");
  d.check_dtype(OperatorId::Add, cpu, DType::F32);
  CHECK_THROWS_WITH(d.check_dtype(OperatorId::Add, cpu, DType::I32), "add: unsupported dtype int32 on cpu");
  bool typed = false;
  try {
    d.select(DispatchRequest{OperatorId::Add, cpu, DType::I64, kContiguous});
  } catch (const UnsupportedOperation&) {
    typed = true;
  }
  CHECK(typed);
  // Observer seam: sees the request and the chosen record.
  std::string seen;
  d.set_observer([&](const DispatchRequest&, const KernelRecord& k) { seen = k.name; });
  OpCall call;
  g_calls = 0;
  d.run(DispatchRequest{OperatorId::Add, cpu, DType::F32, kStrided}, call);
  CHECK_EQ(g_calls, 100);
  CHECK_EQ(seen, std::string("strided"));
}

TEST(builtin_table_is_frozen_and_covers_both_backends) {
  const KernelRegistry& reg = default_dispatcher().registry();
  CHECK(reg.frozen());
  // CPU computes in float32 and float64; CUDA in float32 and the two 16-bit formats.
  for (OperatorId op : {OperatorId::Add, OperatorId::Mul, OperatorId::Matmul, OperatorId::Sum, OperatorId::Relu, OperatorId::Softmax}) {
    CHECK(reg.find(op, Backend::CPU, DType::F32, kContiguous) != nullptr);
    CHECK(reg.find(op, Backend::CPU, DType::F64, kContiguous) != nullptr);
    CHECK(reg.find(op, Backend::CUDA, DType::F32, kContiguous) != nullptr);
    CHECK(reg.find(op, Backend::CUDA, DType::BF16, kContiguous) != nullptr);
    CHECK(reg.find(op, Backend::CUDA, DType::F16, kContiguous) != nullptr);
    CHECK(reg.find(op, Backend::CUDA, DType::F64, kContiguous) == nullptr);
  }
  // Composite operators own no kernels.
  for (OperatorId op : {OperatorId::Sub, OperatorId::Div, OperatorId::Dropout}) {
    CHECK(reg.schema(op).composite);
    for (const KernelRecord& k : reg.kernels()) CHECK(k.op != op);
  }
  CHECK_EQ(std::string(reg.schema(OperatorId::Matmul).name), std::string("matmul"));
  CHECK_EQ(reg.schema(OperatorId::Add).arity, 2);
}

TEST(integer_tensors_are_rejected_by_compute_operators) {
  Tensor a = Tensor::zeros({4}, DType::I64, Device());
  CHECK_THROWS_WITH(ops::add(a, a), "unsupported dtype int64");
  CHECK_THROWS_WITH(ops::relu(a), "unsupported dtype int64");
}

// plan_gemm as a host-only unit (reference project: tests/cpp/test_matmul_planner.cpp).
#include "check.h"
#include "ob/gemm_plan.h"

using namespace ob;

namespace {
GemmProblem problem(DType dt, int64_t m, int64_t n, int64_t k) {
  GemmProblem p;
  p.dtype = dt; p.m = m; p.n = n; p.k = k;
  return p;
}
}  // namespace

TEST(planner_float32_defaults_to_the_fma_kernel) {
  GemmPlanOptions o;
  CHECK(plan_gemm(problem(DType::F32, 4096, 4096, 4096), o).route == GemmRoute::Simt128);
  CHECK(plan_gemm(problem(DType::F32, 64, 64, 64), o).route == GemmRoute::Simt64);
  o.float32_precision = 1;
  CHECK(plan_gemm(problem(DType::F32, 1024, 1024, 1024), o).route == GemmRoute::Tc05Float32);
  GemmProblem with_residual = problem(DType::F32, 1024, 1024, 1024);
  with_residual.has_residual = true;
  CHECK(plan_gemm(with_residual, o).route != GemmRoute::Tc05Float32);
}

TEST(planner_forced_routes) {
  GemmPlanOptions o;
  o.force_route = 1;
  CHECK(plan_gemm(problem(DType::BF16, 8192, 8192, 8192), o).route == GemmRoute::Simt128);
  o.force_route = 2;
  CHECK(plan_gemm(problem(DType::BF16, 16, 16, 16), o).route == GemmRoute::Tc05);
  GemmProblem no_tma = problem(DType::BF16, 1024, 1024, 1024);
  no_tma.tma_ok = false;
  CHECK_THROWS_WITH(plan_gemm(no_tma, o), "cannot take the tcgen05 route");
}

TEST(planner_tile_shapes_on_transformer_products) {
  GemmPlanOptions o;
  GemmPlan p = plan_gemm(problem(DType::BF16, 8192, 6144, 2048), o);
  CHECK(p.route == GemmRoute::Tc05 && p.bn == 256 && p.tm == 256 && p.epilogue_warps == 4);
  p = plan_gemm(problem(DType::BF16, 2048, 2048, 8192), o);
  CHECK(p.route == GemmRoute::Tc05 && p.bn == 256 && p.tm == 128);
  p = plan_gemm(problem(DType::F16, 8192, 8192, 1024), o);
  CHECK(p.tm == 128 && p.epilogue_warps == 8);
  p = plan_gemm(problem(DType::BF16, 512, 512, 16384), o);
  CHECK(p.route == GemmRoute::Tc05SplitK && p.splits == 16);
  o.splitk = false;
  CHECK(plan_gemm(problem(DType::BF16, 512, 512, 16384), o).route == GemmRoute::Tc05);
}

TEST(planner_pairs_are_opt_in_and_described) {
  GemmPlanOptions o;
  CHECK(plan_gemm(problem(DType::BF16, 8192, 8192, 8192), o).route == GemmRoute::Tc05);
  o.pair_mode = 2;
  const GemmPlan p = plan_gemm(problem(DType::BF16, 8192, 8192, 8192), o);
  CHECK(p.route == GemmRoute::Tc05Pair && p.tm == 256 && p.bn == 256);
  CHECK(p.describe().find("tcgen05_pair 512x256") == 0);
  o.pair_mode = 1;
  CHECK(plan_gemm(problem(DType::BF16, 8192, 8192, 2048), o).epilogue_warps == 8);
  CHECK(plan_gemm(problem(DType::BF16, 128, 8192, 2048), o).route == GemmRoute::Tc05);
}

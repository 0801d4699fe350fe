// Host-side planning of one matrix product: which kernel family runs it, with which tile, how
// many epilogue warps, whether the reduction is split, whether CTA pairs are used.  The planner is
// a pure function of the problem description and of the options (which default from the
// environment once per process), so every route can be checked on a machine without a GPU.
// (reference project: include/orthon/planning/matmul_planner.h:8-26, src/planning/matmul_planner.cpp:26-73,
// forced routes of src/diagnostics/matmul.cpp:14-87)
#pragma once

#include <cstdint>
#include <string>

#include "ob/core.h"

namespace ob {

enum class GemmRoute : int {
  Simt64 = 1,        // float32 FMA kernel (also 16-bit operands that TMA cannot describe), 64 x 64 tiles
  Simt128 = 2,       // the register-blocked 128 x 128 form of the same kernel
  Tc05 = 3,          // tcgen05 tiles, one CTA per tile
  Tc05Pair = 4,      // tcgen05 tiles over CTA pairs (cta_group::2)
  Tc05SplitK = 5,    // tcgen05 tiles over K slices with float32 partials and a second pass
  Tc05Float32 = 6,   // float32 operands as bfloat16 pieces on the tensor cores
};

struct GemmProblem {
  DType dtype = DType::BF16;
  int64_t m = 0, n = 0, k = 0;
  int64_t batch = 1;            // product of the batch extents
  bool has_bias = false, has_residual = false, has_preact = false;
  int act = 0;                  // epilogue activation code (0 none, 1 relu, 2 gelu, 3 multiply-by-aux, 4 gelu with derivative)
  bool tma_ok = true;           // both operands can be described by tensor maps (after packing, if needed)
  bool tcgen05 = true;          // the device has 5th-generation tensor cores
  int sms = 148;
};

struct GemmPlanOptions {
  int force_route = 0;          // 0 planner decides, 1 force the SIMT kernel, 2 require tcgen05
  int float32_precision = 0;    // 0 "highest" (exact FMA), 1 "high" (bfloat16 pieces for large products)
  long long float32_split_min = 1LL << 22;
  int force_bn = 0;             // 128 / 256 forces the tile width
  int force_tm = 0;             // 128 / 256 forces the tile height
  int tall_min_k = 2048;        // 256-row tiles from this reduction length on
  int ew8_max_k = 1024;         // eight epilogue warps up to this reduction length (128 x 256 tile)
  bool splitk = true;
  int pair_mode = -1;           // -1 planner decides, 0 never, 1 256 x 256 pair tiles, 2 512 x 256 pair tiles
  int pair_ew8_max_k = 4096;
  bool tall_preact = true;      // 256-row tiles also for epilogues that store a second output
  static GemmPlanOptions from_environment();
};

struct GemmPlan {
  GemmRoute route = GemmRoute::Simt64;
  int bn = 0, tm = 0;           // CTA tile (columns, rows); for pairs the pair covers 2 tm rows
  int epilogue_warps = 4;
  int splits = 1;               // K slices (Tc05SplitK)
  const char* why = "";         // one phrase for diagnostics
  std::string describe() const;
};

// Throws std::runtime_error when `force_route == 2` and the problem cannot take the tensor-core route.
GemmPlan plan_gemm(const GemmProblem& p, const GemmPlanOptions& o);

}  // namespace ob

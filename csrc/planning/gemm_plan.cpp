// plan_gemm: see ob/gemm_plan.h.  Thresholds are measurements on B200 (sustained, power-capped
// throughput of the candidate tiles on transformer shapes); each rule says what it trades.
#include "ob/gemm_plan.h"

#include <cstdlib>
#include <stdexcept>

namespace ob {

namespace {
int env_int(const char* name, int fallback) {
  const char* e = std::getenv(name);
  return (e != nullptr && *e != '\0') ? std::atoi(e) : fallback;
}
long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
}  // namespace

GemmPlanOptions GemmPlanOptions::from_environment() {
  GemmPlanOptions o;
  const char* f32 = std::getenv("ORTHON_FLOAT32_MATMUL");
  o.float32_precision = (f32 != nullptr && std::string(f32) == "high") ? 1 : 0;
  const char* split_min = std::getenv("ORTHON_GEMM_F32_SPLIT_MIN");
  if (split_min != nullptr) o.float32_split_min = std::atoll(split_min);
  o.force_bn = env_int("ORTHON_GEMM_BN", 0);
  o.force_tm = env_int("ORTHON_GEMM_TM", 0);
  o.tall_min_k = env_int("ORTHON_GEMM_TALL_MIN_K", o.tall_min_k);
  o.ew8_max_k = env_int("ORTHON_GEMM_EW8_MAX_K", o.ew8_max_k);
  o.splitk = env_int("ORTHON_GEMM_SPLITK", 1) != 0;
  o.pair_mode = env_int("ORTHON_GEMM_PAIR", o.pair_mode);
  o.pair_ew8_max_k = env_int("ORTHON_GEMM_PAIR_EW8_MAX_K", o.pair_ew8_max_k);
  o.tall_preact = env_int("ORTHON_GEMM_TALL_PREACT", 1) != 0;
  return o;
}

std::string GemmPlan::describe() const {
  static const char* names[] = {"none", "simt_64x64", "simt_128x128", "tcgen05", "tcgen05_pair", "tcgen05_split_k", "tcgen05_float32"};
  std::string s = names[static_cast<int>(route)];
  if (route >= GemmRoute::Tc05) {
    s += " " + std::to_string(route == GemmRoute::Tc05Pair ? 2 * tm : tm) + "x" + std::to_string(bn);
    s += " ew" + std::to_string(epilogue_warps);
    if (splits > 1) s += " splits " + std::to_string(splits);
  }
  return s + " (" + why + ")";
}

static GemmPlan simt_plan(const GemmProblem& p, const char* why) {
  // Large tiles once they fill the GPU at least once over; short reductions do not amortise the
  // 64-register prologue / epilogue of the large tile, small problems want the parallelism.
  GemmPlan plan;
  const long long big_tiles = ceil_div(p.n, 128) * ceil_div(p.m, 128) * p.batch;
  const bool big = p.m >= 128 && p.n >= 128 && p.k >= 256 && big_tiles >= p.sms;
  plan.route = big ? GemmRoute::Simt128 : GemmRoute::Simt64;
  plan.bn = plan.tm = big ? 128 : 64;
  plan.why = why;
  return plan;
}

GemmPlan plan_gemm(const GemmProblem& p, const GemmPlanOptions& o) {
  if (p.dtype == DType::F32) {
    // "high" precision: large products as six bfloat16 piece products on the tensor cores; small
    // ones, and epilogues with a residual or a stored pre-activation, stay on the FMA kernel.
    const bool can_split = p.tcgen05 && !p.has_residual && !p.has_preact && p.act <= 2 && p.k * 6 + 8 < (1LL << 31);
    const bool split = can_split && o.force_route != 1 &&
                       (o.force_route == 2 || (o.float32_precision == 1 && p.m * p.n * p.k >= o.float32_split_min));
    if (!split) {
      if (o.force_route == 2) throw std::runtime_error("matmul diagnostics: this float32 problem cannot take the tcgen05 route");
      return simt_plan(p, o.force_route == 1 ? "forced" : "float32 is exact FMA arithmetic by default");
    }
    GemmPlan plan;
    plan.route = GemmRoute::Tc05Float32;
    plan.bn = p.n > 128 ? 256 : 128;
    plan.tm = 128;
    plan.why = "float32 as bfloat16 pieces";
    return plan;
  }
  const bool tiny = p.m * p.n * p.k < (1LL << 18) && o.force_route != 2;
  if (tiny || o.force_route == 1 || !p.tcgen05 || !p.tma_ok) {
    if (o.force_route == 2) throw std::runtime_error("matmul diagnostics: this problem cannot take the tcgen05 route");
    return simt_plan(p, tiny ? "too small to fill one tensor-core tile wave" : (o.force_route == 1 ? "forced" : "operands are not TMA-describable"));
  }
  GemmPlan plan;
  const bool plain = !p.has_bias && !p.has_residual && !p.has_preact && p.act == 0;
  const long long tiles_wide = ceil_div(p.m, 128) * ceil_div(p.n, 256);
  // Split-K: a small output with a long reduction (weight gradients of a narrow model) gives the
  // persistent grid a handful of tiles; the reduction is cut into slices that run as batch entries.
  if (o.splitk && plain && p.batch == 1 && p.n % 4 == 0 && tiles_wide * 4 <= p.sms && p.k >= 4096) {
    int splits = 1;
    while (splits < 32 && tiles_wide * splits * 2 <= p.sms && p.k % (splits * 2 * 64) == 0 && p.k / (splits * 2) >= 512) splits *= 2;
    if (splits > 1) {
      plan.route = GemmRoute::Tc05SplitK;
      plan.splits = splits;
      plan.bn = (p.n > 128 && tiles_wide * splits * 2 > p.sms) ? 256 : 128;
      plan.tm = 128;
      plan.why = "few output tiles, long reduction";
      return plan;
    }
  }
  // Tile width: 256 columns whenever the problem is wider than one 128-column tile, unless that
  // would leave at least half of the SMs without a tile (narrow tiles run at two thirds of the
  // wide tile's rate, so they pay only when twice as many of them still fit in one wave).
  bool wide = p.n > 128;
  if (o.force_bn == 128 || (o.force_bn != 256 && wide && tiles_wide * p.batch * 2 <= p.sms)) wide = false;
  plan.route = GemmRoute::Tc05;
  plan.bn = wide ? 256 : 128;
  plan.tm = 128;
  plan.why = wide ? "wide tile" : "narrow tile fills more SMs";
  // 256-row tiles (two MMA row blocks per B stage) when the reduction is long enough to amortise
  // their epilogue, which overlaps the next tile only partly, and the waves fill to 80 %.
  const long long tiles256 = ceil_div(p.m, 256) * ceil_div(p.n, 256) * p.batch;
  const double eff256 = static_cast<double>(tiles256) / static_cast<double>(ceil_div(tiles256, p.sms) * p.sms);
  // A second output (stored pre-activation) goes through the same staging tile after the result,
  // which lengthens the epilogue; the tile still pays (measured on the first MLP product of the
  // 1.3 B model).  ORTHON_GEMM_TALL_PREACT=0 keeps such products on the 128-row tile.
  const bool tall = wide && o.force_tm != 128 && (!p.has_preact || o.tall_preact) &&
                    (o.force_tm == 256 || (p.m >= 512 && p.k >= o.tall_min_k && eff256 >= 0.8));
  // CTA pairs.  Measured under the power cap (1.3 B transformer shapes, 8192 tokens) the pair tiles
  // tie with the single-CTA 256 x 256 tile wherever that one is eligible, so the planner keeps the
  // single-CTA tile there.  Where it is not (a long reduction over an output whose 256 x 256
  // tiling fills its waves badly: the weight gradient of a fused QKV projection, 2048 x 6144 over
  // 8192 tokens) the 256 x 256 pair tile, whose epilogue overlaps the next main loop, beats the
  // 128 x 256 tile by a tenth (1088 against 990 TFLOP/s).  pair_mode 1 / 2 force pairs everywhere.
  const bool pair_auto = o.pair_mode < 0 && wide && !tall && p.m >= 256 && p.k >= 4096 && !p.has_preact &&
                         ceil_div(p.m, 256) * ceil_div(p.n, 256) * p.batch > p.sms / 2;
  const bool pair = wide && p.m >= 256 && (o.pair_mode >= 1 || pair_auto);
  if (pair) {
    plan.route = GemmRoute::Tc05Pair;
    const bool pair_tall = o.pair_mode == 2 && p.m >= 512 && !p.has_preact;
    plan.tm = pair_tall ? 256 : 128;
    plan.epilogue_warps = (!pair_tall && p.k <= o.pair_ew8_max_k && !p.has_preact) ? 8 : 4;
    plan.why = pair_tall ? "512 x 256 pair tile" : "256 x 256 pair tile";
    return plan;
  }
  if (tall) {
    plan.tm = 256;
    plan.why = "long reduction: two row blocks share each B stage";
    return plan;
  }
  // Short reductions: the epilogue, not the MMA loop, sets the pace of a tile; eight warps drain it.
  if (wide && p.k <= o.ew8_max_k && !p.has_preact) {
    plan.epilogue_warps = 8;
    plan.why = "short reduction: eight epilogue warps";
  }
  return plan;
}

}  // namespace ob

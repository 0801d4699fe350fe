// Planner of the implicit-GEMM convolution launches (see ob/conv_plan.h).
#include "ob/conv_plan.h"

#include <algorithm>

namespace ob {

namespace {
int round16(int v) { return (v + 15) & ~15; }
int round1k(int v) { return (v + 1023) & ~1023; }

// Ring geometry: as many slots as fit (2 to 4), kept under half of the shared memory when three
// slots allow it, so that two CTAs share an SM and one's gathers hide the other's waits.
void plan_ring(ConvPlan& p) {
  const int rows_bytes = round1k(p.bn * 128);
  const bool wgrad = p.pass == ConvPass::WeightGradient;
  p.gather_bytes = wgrad ? rows_bytes : 16384;
  p.stage_bytes = p.gather_bytes + (wgrad ? 16384 : rows_bytes);
  const int half = 110 * 1024, whole = kConvPlanSmemMax - 2048;
  const int budget = 3 * p.stage_bytes <= half ? half : whole;
  p.stages = std::max(2, std::min(kConvPlanMaxStages, budget / p.stage_bytes));
  int cols = 32;
  while (cols < p.bn) cols *= 2;
  p.tmem_cols = cols;
  p.smem_bytes = p.stages * p.stage_bytes + 1024 + 256;
  // Registers allow two CTAs per SM; shared memory and the 512 columns of tensor memory decide.
  p.ctas_per_sm = std::max(1, std::min({2, kConvPlanSmemMax / (p.smem_bytes + 1024), 512 / p.tmem_cols}));
}

void finish(ConvPlan& p, int sms) {
  p.grid = static_cast<int>(std::max<long long>(1, std::min<long long>(p.items, static_cast<long long>(sms) * p.ctas_per_sm)));
}
}  // namespace

std::string ConvPlan::describe() const {
  if (!eligible) return std::string("not eligible: ") + why;
  static const char* names[] = {"forward", "input gradient", "weight gradient"};
  std::string s = names[static_cast<int>(pass)];
  s += " bn" + std::to_string(bn) + " tiles " + std::to_string(tiles_m) + "x" + std::to_string(tiles_n);
  if (classes > 1) s += " classes " + std::to_string(classes);
  if (splits > 1) s += " splits " + std::to_string(splits);
  s += " ring " + std::to_string(stages) + "x" + std::to_string(stage_bytes) + " grid " + std::to_string(grid);
  s += fast ? " row-uniform gather" : " per-element gather";
  return s;
}

ConvPlan plan_conv(ConvPass pass, const ConvGeometry& g, int sms) {
  ConvPlan p;
  p.pass = pass;
  if (g.N < 1 || g.C < 1 || g.K < 1 || g.R < 1 || g.S < 1 || g.sh < 1 || g.sw < 1 || g.ph < 0 || g.pw < 0 ||
      g.H + 2 * g.ph < g.R || g.W + 2 * g.pw < g.S) {
    p.why = "invalid geometry";
    return p;
  }
  p.out_h = g.out_h(); p.out_w = g.out_w();
  const long long lim = (1LL << 31) - 1;
  const long long P = static_cast<long long>(p.out_h) * p.out_w;
  if (static_cast<long long>(g.N) * g.C * g.H * g.W >= lim || static_cast<long long>(g.N) * g.K * P >= lim) {
    p.why = "tensor offsets do not fit 32 bits";
    return p;
  }
  if (sms < 1) sms = 1;
  const int CRS = g.C * g.R * g.S;
  if (pass == ConvPass::Forward) {
    p.rows_total = CRS;
    p.weight_ld = (CRS + 7) & ~7;
    p.pad_weights = p.weight_ld != CRS;
    p.bn = std::min(256, round16(g.K));
    p.tiles_m = static_cast<int>((static_cast<long long>(g.N) * P + 127) / 128);
    p.tiles_n = (g.K + p.bn - 1) / p.bn;
    p.items = static_cast<long long>(p.tiles_m) * p.tiles_n;
    p.fast = g.S <= 8 && p.out_w % 8 == 0;
  } else if (pass == ConvPass::InputGradient) {
    p.classes = g.sh * g.sw;
    const int taps_max = ((g.R + g.sh - 1) / g.sh) * ((g.S + g.sw - 1) / g.sw);
    p.weight_ld = (g.K * taps_max + 7) & ~7;
    p.zero_fill = g.sh > g.R || g.sw > g.S;
    p.bn = std::min(256, round16(g.C));
    const long long m_class = static_cast<long long>(g.N) * ((g.H + g.sh - 1) / g.sh) * ((g.W + g.sw - 1) / g.sw);   // class (0, 0) is the largest
    p.tiles_m = static_cast<int>((m_class + 127) / 128);
    p.tiles_n = (g.C + p.bn - 1) / p.bn;
    p.items = static_cast<long long>(p.tiles_m) * p.tiles_n * p.classes;
    p.fast = g.S <= 8 && g.W % (8 * g.sw) == 0;
  } else {
    if (g.K > 128) { p.why = "more than 128 output channels (one 128-row tile of the output gradient)"; return p; }
    if (P % 8 != 0) { p.why = "output plane is not a multiple of 8 pixels (TMA row pitch)"; return p; }
    const int rows = CRS + 1;   // + the column of ones that yields the bias gradient
    p.rows_total = rows;
    p.tiles_m = 1;
    p.tiles_n = (rows + 255) / 256;
    p.bn = round16((rows + p.tiles_n - 1) / p.tiles_n);
    p.fast = g.S <= 8 && p.out_w % 8 == 0;
  }
  plan_ring(p);
  if (pass == ConvPass::WeightGradient) {
    const long long kb_img = (P + 63) / 64;
    p.kb_total = static_cast<long long>(g.N) * kb_img;
    // One wave of (column tile, reduction slice) items, and no more than one slice per four blocks of 64 pixels.
    int splits = static_cast<int>(std::max<long long>(1, std::min<long long>((p.kb_total + 3) / 4, (static_cast<long long>(sms) * p.ctas_per_sm) / p.tiles_n)));
    p.kb_per_split = static_cast<int>((p.kb_total + splits - 1) / splits);
    p.splits = static_cast<int>((p.kb_total + p.kb_per_split - 1) / p.kb_per_split);
    p.ldp = p.tiles_n * p.bn;
    p.items = static_cast<long long>(p.tiles_n) * p.splits;
  }
  finish(p, sms);
  p.eligible = true;
  p.why = p.fast ? "row-uniform gather" : "per-element gather";
  return p;
}

}  // namespace ob

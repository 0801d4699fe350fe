// plan_conv and the stride-class geometry as host-only units.
#include <vector>

#include "check.h"
#include "ob/conv_plan.h"

using namespace ob;

namespace {
ConvGeometry layer(int N, int C, int H, int W, int K, int R, int S, int stride, int pad) {
  ConvGeometry g;
  g.N = N; g.C = C; g.H = H; g.W = W; g.K = K; g.R = R; g.S = S; g.sh = g.sw = stride; g.ph = g.pw = pad;
  return g;
}
}  // namespace

TEST(conv_plan_forward_of_the_small_cnn_layers) {
  const ConvPlan a = plan_conv(ConvPass::Forward, layer(128, 3, 32, 32, 32, 3, 3, 1, 1), 148);
  CHECK(a.eligible && a.fast && a.bn == 32 && a.tiles_m == 1024 && a.tiles_n == 1 && a.rows_total == 27);
  CHECK(a.pad_weights && a.weight_ld == 32 && a.ctas_per_sm == 2 && a.grid == 296 && a.stages == 4);
  const ConvPlan b = plan_conv(ConvPass::Forward, layer(128, 64, 16, 16, 128, 3, 3, 2, 1), 148);
  CHECK(b.eligible && b.fast && b.bn == 128 && b.tiles_m == 64 && !b.pad_weights && b.weight_ld == 576);
  CHECK(b.grid == 64 && b.out_h == 8 && b.out_w == 8);
}

TEST(conv_plan_input_gradient_splits_the_pixels_by_stride_class) {
  const ConvGeometry g = layer(128, 32, 32, 32, 64, 3, 3, 2, 1);
  const ConvPlan p = plan_conv(ConvPass::InputGradient, g, 148);
  CHECK(p.eligible && p.classes == 4 && p.fast && !p.zero_fill && p.bn == 32);
  CHECK(p.tiles_m == 128 * 16 * 16 / 128 && p.items == static_cast<long long>(p.tiles_m) * 4);
  int taps = 0, pixels = 0;
  for (int z = 0; z < p.classes; ++z) {
    const StrideClass c = stride_class_of(z, g.H, g.W, g.R, g.S, g.sh, g.sw, g.ph, g.pw);
    taps += c.ra * c.sb;
    pixels += c.ha * c.wb;
  }
  CHECK(taps == 9);          // every filter tap is seen by exactly one class
  CHECK(pixels == 32 * 32);  // every input pixel belongs to exactly one class
}

TEST(conv_plan_stride_classes_reproduce_the_direct_index_formula) {
  for (int stride = 1; stride <= 3; ++stride)
    for (int pad = 0; pad <= 2; ++pad)
      for (int R = 1; R <= 5; R += 2) {
        const int H = 11;
        for (int z = 0; z < stride * stride; ++z) {
          const StrideClass c = stride_class_of(z, H, H, R, R, stride, stride, pad, pad);
          for (int i = 0; i < c.ha; ++i)
            for (int ri = 0; ri < c.ra; ++ri) {
              const int ih = c.a + stride * i, r = c.ra0 + stride * ri;
              CHECK((ih + pad - r) % stride == 0);
              CHECK((ih + pad - r) / stride == i + c.qa - ri);
            }
        }
      }
}

TEST(conv_plan_stride_larger_than_the_filter_asks_for_a_zero_fill) {
  const ConvPlan p = plan_conv(ConvPass::InputGradient, layer(2, 8, 8, 8, 16, 1, 1, 2, 0), 148);
  CHECK(p.eligible && p.zero_fill && p.classes == 4);
  CHECK(!plan_conv(ConvPass::InputGradient, layer(2, 8, 8, 8, 16, 3, 3, 2, 1), 148).zero_fill);
}

TEST(conv_plan_weight_gradient_slices_and_eligibility) {
  const ConvPlan p = plan_conv(ConvPass::WeightGradient, layer(128, 32, 32, 32, 64, 3, 3, 2, 1), 148);
  CHECK(p.eligible && p.rows_total == 289 && p.tiles_n == 2 && p.bn == 160 && p.ldp == 320);
  CHECK(p.kb_total == 128 * 4 && static_cast<long long>(p.splits) * p.kb_per_split >= p.kb_total);
  CHECK(static_cast<long long>(p.splits - 1) * p.kb_per_split < p.kb_total);
  const ConvPlan wide = plan_conv(ConvPass::WeightGradient, layer(2, 6, 10, 10, 130, 3, 3, 1, 1), 148);
  CHECK(!wide.eligible && std::string(wide.why).find("128") != std::string::npos);
  const ConvPlan odd = plan_conv(ConvPass::WeightGradient, layer(3, 4, 9, 11, 20, 3, 3, 2, 0), 148);
  CHECK(!odd.eligible && std::string(odd.why).find("8 pixels") != std::string::npos);
}

TEST(conv_plan_ring_never_exceeds_the_sm) {
  for (int K : {8, 32, 64, 128, 200, 512})
    for (int C : {3, 16, 64, 256}) {
      for (ConvPass pass : {ConvPass::Forward, ConvPass::InputGradient, ConvPass::WeightGradient}) {
        const ConvPlan p = plan_conv(pass, layer(4, C, 16, 16, K, 3, 3, 1, 1), 148);
        if (!p.eligible) continue;
        CHECK(p.stages >= 2 && p.stages <= kConvPlanMaxStages);
        CHECK(p.smem_bytes <= kConvPlanSmemMax);
        CHECK(p.ctas_per_sm * p.tmem_cols <= 512);
        CHECK(p.bn % 16 == 0 && p.bn <= 256 && p.tmem_cols >= p.bn);
      }
    }
}

TEST(conv_plan_refuses_bad_geometry) {
  CHECK(!plan_conv(ConvPass::Forward, layer(1, 1, 2, 2, 1, 3, 3, 1, 0), 148).eligible);
  CHECK(!plan_conv(ConvPass::Forward, layer(0, 1, 8, 8, 1, 3, 3, 1, 1), 148).eligible);
  CHECK(!plan_conv(ConvPass::Forward, layer(4096, 1024, 32, 32, 8, 1, 1, 1, 0), 148).eligible);
}

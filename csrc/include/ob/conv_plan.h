// Host-side planning of one implicit-GEMM convolution launch (forward, input gradient or weight
// gradient): tile counts, stride classes, reduction slices, the ring of operand slots and the
// grid.  A pure function of the layer's geometry and the SM count, so the index arithmetic that
// the kernel relies on can be checked on a machine without a GPU.  The stride-class geometry is
// shared with the kernel (same inline function on both sides).
// (reference project: the selectors of src/backends/cuda/conv2d_cuda.cu:1173-1202, :1778-1812 and
// the diagnostics of src/diagnostics/conv2d.cpp play this role there)
#pragma once

#include <string>

#if defined(__CUDACC__)
#define OB_HD __host__ __device__
#else
#define OB_HD
#endif

namespace ob {

struct ConvGeometry {
  int N = 0, C = 0, H = 0, W = 0;   // input [N, C, H, W]
  int K = 0, R = 0, S = 0;          // filter [K, C, R, S]
  int sh = 1, sw = 1, ph = 0, pw = 0;
  int out_h() const { return (H + 2 * ph - R) / sh + 1; }
  int out_w() const { return (W + 2 * pw - S) / sw + 1; }
};

// Input gradient, stride class z = a * sw + b: the input pixels (a + sh*i, b + sw*j).  They are
// reached only by the filter rows r = ra0 + sh*ri (ri < ra) and columns s = sb0 + sw*si (si < sb);
// the class has ha x wb pixels per image; output pixel (i + qa - ri, j + qb - si) feeds pixel (i, j)
// of the class through tap (ri, si).
struct StrideClass {
  int a, b, ra0, sb0, ra, sb, ha, wb, qa, qb;
};
OB_HD inline StrideClass stride_class_of(int z, int H, int W, int R, int S, int sh, int sw, int ph, int pw) {
  StrideClass c;
  c.a = z / sw; c.b = z - c.a * sw;
  c.ra0 = (c.a + ph) % sh; c.sb0 = (c.b + pw) % sw;
  c.ra = c.ra0 < R ? (R - c.ra0 + sh - 1) / sh : 0;
  c.sb = c.sb0 < S ? (S - c.sb0 + sw - 1) / sw : 0;
  c.ha = c.a < H ? (H - c.a + sh - 1) / sh : 0;
  c.wb = c.b < W ? (W - c.b + sw - 1) / sw : 0;
  c.qa = (c.a + ph) / sh; c.qb = (c.b + pw) / sw;
  return c;
}

enum class ConvPass : int { Forward = 0, InputGradient = 1, WeightGradient = 2 };

struct ConvPlan {
  bool eligible = false;
  const char* why = "";          // one phrase: why not, or which gather
  ConvPass pass = ConvPass::Forward;
  int out_h = 0, out_w = 0;
  int rows_total = 0;            // forward: C*R*S taps; weight gradient: C*R*S + 1 gathered rows; input gradient: per class (0 here)
  int bn = 0;                    // MMA N (multiple of 16, at most 256)
  int tiles_m = 0, tiles_n = 0;  // 128-pixel tiles (input gradient: of the largest class), column tiles
  int classes = 1;               // input gradient: sh * sw
  int weight_ld = 0;             // row length of the (padded / permuted) weight matrix, a multiple of 8
  bool pad_weights = false;      // forward: the weight rows need a padded copy for TMA
  bool zero_fill = false;        // input gradient: some pixels are reached by no tap
  int splits = 1, kb_per_split = 0;   // weight gradient: reduction slices, 64-pixel blocks per slice
  long long kb_total = 0;             // weight gradient: 64-pixel blocks in the whole reduction
  int ldp = 0;                   // weight gradient: row length of the float32 partials
  bool fast = false;             // row-uniform gather (groups of 8 pixels share an output row)
  int gather_bytes = 0, stage_bytes = 0, stages = 0, tmem_cols = 0;
  int smem_bytes = 0, ctas_per_sm = 1;
  long long items = 0;           // work items a persistent grid walks
  int grid = 0;
  std::string describe() const;
};

constexpr int kConvPlanSmemMax = 227 * 1024;
constexpr int kConvPlanMaxStages = 4;

ConvPlan plan_conv(ConvPass pass, const ConvGeometry& g, int sms);

}  // namespace ob

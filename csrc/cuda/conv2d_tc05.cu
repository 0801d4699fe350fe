// conv2d as an implicit GEMM on the 5th-generation tensor cores (sm_100a): the unfolded
// (im2col) matrix never exists in memory.  The warps of a CTA gather the rows of it that the
// current 64-wide reduction block needs straight from the NCHW activations into the
// 128-byte-swizzled shared-memory layout that tcgen05.mma reads, the other operand arrives by
// TMA, accumulators live in tensor memory.
//
//   fprop  out[n, k, oh, ow] = sum_{c,r,s} x[n, c, oh*sh-ph+r, ow*sw-pw+s] * w[k, c, r, s] + b[k]
//          M = N*OH*OW output pixels (128 per tile), N = K channels, reduction C*R*S.
//          A (gathered, pixel-contiguous = MN-major) x B (weights [K, CRS], TMA, K-major).
//   dgrad  dx[n, c, ih, iw] = sum_{k,r,s} gy[n, k, (ih+ph-r)/sh, (iw+pw-s)/sw] * w[k, c, r, s]
//          done per stride class (ih mod sh, iw mod sw): the pixels of a class see only the filter
//          rows r = ra0 + sh*ri and columns s = sb0 + sw*si, so nothing is multiplied by the zeros a
//          strided convolution leaves between its taps, and no index is divided in the inner loop.
//          M = pixels of the class, N = C channels, reduction K * taps of the class.
//          A (gathered from gy, MN-major) x B (weights permuted per class to [C, K*taps], TMA).
//   wgrad  dw[k, (c,r,s)] = sum_{n,oh,ow} gy[n, k, oh, ow] * x[n, c, oh*sh-ph+r, ow*sw-pw+s]
//          M = K channels, N = C*R*S (+ one column of ones whose result is the bias gradient),
//          reduction N*OH*OW pixels cut into slices (split-K) with float32 partials and a fixed-order
//          second pass.  A (gy, TMA, K-major) x B (gathered, K-major).
//
// In all three the gathered tile is "rows of 64 consecutive pixels": row = one (c, r, s) (or
// (k, ri, si)) tap, 128 bytes, chunk c of row q stored at q * 128 + ((c ^ (q & 7)) << 4), which is
// both the MN-major A layout (fprop, dgrad) and the K-major B layout (wgrad) of a 128-byte-swizzled
// tile.  CTAs are persistent (a grid of at most two per SM walks the work items; the ring of
// operand slots and its barrier phases run on across items).  When output rows are a multiple of 8
// pixels a thread's 8 pixels share one row: one vertical test and one precomputed column mask then
// cover 8 loads (FAST); other shapes take a per-element path.  Every mbarrier wait is bounded.
// bfloat16 and float16; float32 stays on the GEMM lowering.
//
// Replaces (reference project paths): src/backends/cuda/conv2d_cuda.cu:311-2121 (tiled forward,
// input-gradient and weight-gradient kernels and their selectors :1173-1202, :1778-1812).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "ob/conv_plan.h"
#include "ob/cuda_common.cuh"
#include "ob/ops.h"
#include "ob/tc05.cuh"

namespace ob {
namespace cu {

int* tc05_error_flag(int device);
bool tc05_encode_map(CUtensorMap* out, DType dt, int rank, void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box);

namespace {

using namespace tc05;

constexpr int kConvThreads = 256;
constexpr int kMaxStages = kConvPlanMaxStages;
constexpr int kConvSmemMax = kConvPlanSmemMax;
enum : int { kErrConvWait = 21 };

struct ConvParams {
  int mode;                    // 0 fprop, 1 dgrad, 2 wgrad
  int N, C, H, W, K, R, S, OH, OW, sh, sw, ph, pw;
  int rows_total;              // fprop: C*R*S reduction taps; wgrad: gathered rows (C*R*S + 1); dgrad: per class, computed in the kernel
  int bn;                      // MMA N of this launch (multiple of 16, <= 256)
  int tiles_m, tiles_n;        // fprop / dgrad: 128-pixel tiles (dgrad: of the largest class) and column tiles; wgrad: tiles_n only
  int classes;                 // dgrad: sh * sw stride classes; otherwise 1
  int splits, kb_per_split;    // wgrad: reduction slices and 64-pixel blocks per slice
  const void* src;             // gathered source: x (fprop, wgrad) or gy (dgrad)
  void* out;                   // fprop: out, dgrad: dx, wgrad: float32 partials [splits][128][ldp]
  const void* bias;            // fprop
  int ldp;                     // wgrad: row length of the partials
  int gather_bytes, stage_bytes, stages;   // one ring slot = gathered tile then TMA tile (both multiples of 1024 bytes)
  int tmem_cols;               // accumulator columns to allocate: a power of two >= max(32, bn)
  int* err;
};

// One of the 8 consecutive pixels a thread gathers: element offset of its window corner in channel
// plane 0 of its image, and the corner's coordinates (a pixel that does not exist gets a row far
// outside the plane, so every bounds test on it fails).
struct Pix {
  int off, y, x;
};
constexpr int kNoPixel = -(1 << 28);

// How the gathered operand is addressed.  Element (plane a, tap offsets dy, dx) of pixel q is
//   src[q.off + a * plane + dy * rowlen + dx]   if 0 <= q.y + dy < ylim and 0 <= q.x + dx < xlim, else 0.
// fprop / wgrad gather x: plane = H*W, taps add (r, s).  dgrad gathers gy for one stride class:
// plane = OH*OW, taps subtract (ri, si).
struct GatherGeom {
  int plane, rowlen, ylim, xlim, sign;   // sign = +1 (taps add) or -1 (taps subtract)
  int tr, ts;                            // taps per plane: tr x ts
};

template <class T>
__device__ __forceinline__ T gather_one(const T* __restrict__ src, const GatherGeom& g, const Pix& q, int base, int dy, int dx) {
  const bool ok = static_cast<unsigned>(q.y + dy) < static_cast<unsigned>(g.ylim) && static_cast<unsigned>(q.x + dx) < static_cast<unsigned>(g.xlim);
  return ok ? src[q.off + base] : from_f<T>(0.f);
}

__device__ __forceinline__ StrideClass stride_class(const ConvParams& p, int z) {
  return stride_class_of(z, p.H, p.W, p.R, p.S, p.sh, p.sw, p.ph, p.pw);
}

// ---- the fast gather: 8 consecutive pixels that share an image and an output row
// When the row length is a multiple of 8 every aligned group of 8 pixels has one window-corner row
// y0, corner columns x0 + e * step and is wholly inside or wholly outside the problem.  Whether
// column e is inside for horizontal tap tj does not depend on the plane or the vertical tap, so it
// is worked out once per group: bit 8 * tj + e of `xm`.  A row of the gathered tile is then one
// vertical test, one mask byte and 8 predicated loads at fixed offsets from one pointer.
template <class T>
struct Chunk {
  const T* ptr;              // element under the window corner of pixel 0 in plane 0 (may point outside: only masked-in elements are read)
  int y0;                    // corner row; kNoPixel for a group past the end of the problem
  unsigned long long xm;
};
template <class T>
__device__ __forceinline__ Chunk<T> make_chunk(const T* src, bool exists, int off0, int y0, int x0, int step, const GatherGeom& g) {
  Chunk<T> c{src + off0, exists ? y0 : kNoPixel, 0ull};
  for (int tj = 0; tj < g.ts; ++tj) {
    unsigned m = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) m |= (static_cast<unsigned>(x0 + e * step + g.sign * tj) < static_cast<unsigned>(g.xlim) ? 1u : 0u) << e;
    c.xm |= static_cast<unsigned long long>(m) << (8 * tj);
  }
  return c;
}
template <class T>
__device__ __forceinline__ uint4 gather8(const T* q, unsigned m, int step) {
  Pack<T> pk;
  const T zero = from_f<T>(0.f);
  if (step == 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) pk.v[e] = (m >> e) & 1u ? q[e] : zero;
  } else if (step == 2) {
#pragma unroll
    for (int e = 0; e < 8; ++e) pk.v[e] = (m >> e) & 1u ? q[2 * e] : zero;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) pk.v[e] = (m >> e) & 1u ? q[e * step] : zero;
  }
  return *reinterpret_cast<uint4*>(&pk);
}
// A tap index as digits (plane a, vertical ti, horizontal tj) that is advanced by a fixed stride
// without dividing.
struct TapCursor {
  int tap, a, ti, tj;
};
__device__ __forceinline__ TapCursor tap_cursor(int tap, const GatherGeom& g) {
  const int per_plane = g.tr * g.ts;
  TapCursor c;
  c.tap = tap; c.a = tap / per_plane;
  const int t2 = tap - c.a * per_plane;
  c.ti = t2 / g.ts; c.tj = t2 - c.ti * g.ts;
  return c;
}
__device__ __forceinline__ void advance(TapCursor& c, const TapCursor& by, const GatherGeom& g) {
  c.tap += by.tap;
  c.tj += by.tj;
  if (c.tj >= g.ts) { c.tj -= g.ts; ++c.ti; }
  c.ti += by.ti;
  if (c.ti >= g.tr) { c.ti -= g.tr; ++c.a; }
  c.a += by.a;
}
template <class T>
__device__ __forceinline__ uint4 gather_row(const Chunk<T>& ch, const TapCursor& c, bool live, int step, const GatherGeom& g) {
  const bool y_ok = static_cast<unsigned>(ch.y0 + g.sign * c.ti) < static_cast<unsigned>(g.ylim);
  const unsigned m = (live && y_ok) ? static_cast<unsigned>(ch.xm >> (8 * c.tj)) & 0xffu : 0u;
  return gather8<T>(ch.ptr + (c.a * g.plane + g.sign * (c.ti * g.rowlen + c.tj)), m, step);
}

template <class T, int MODE, bool FAST>
__global__ void __launch_bounds__(kConvThreads, 2)
conv_tc05_kernel(const __grid_constant__ CUtensorMap map_t, ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.stages * p.stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* done_bar = empty_bar + kMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int mode = MODE;
  const T* src = static_cast<const T*>(p.src);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], kConvThreads + 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(done_bar, 1);
    mbar_init_fence();
  }
  if (warp == 4) tmem_alloc(tmem_slot, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int P = p.OH * p.OW, HW = p.H * p.W;
  const int kb_img = (P + 63) / 64;                            // wgrad: 64-pixel blocks per image
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  // A is MN-major for fprop / dgrad (gathered, pixels contiguous) and K-major for wgrad (TMA); B is K-major.
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((mode != 2 ? 1u : 0u) << 15) | (static_cast<uint32_t>(p.bn >> 3) << 17) |
                         (static_cast<uint32_t>(128 >> 4) << 24);
  const long long items = mode == 2 ? static_cast<long long>(p.tiles_n) * p.splits
                                    : static_cast<long long>(p.tiles_m) * p.tiles_n * p.classes;
  int stage = 0;                           // ring slot and its phase run on across items
  uint32_t phase = 0;
  unsigned tile_count = 0;
  bool ok = true;

  for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
    // ---- which part of the problem this item is
    int z = 0, tile_m = 0, tile_n = 0, split = 0;
    if (mode == 2) {
      split = static_cast<int>(item / p.tiles_n);
      tile_n = static_cast<int>(item - static_cast<long long>(split) * p.tiles_n);
    } else {
      const int per_class = p.tiles_m * p.tiles_n;
      z = static_cast<int>(item / per_class);
      const int rest = static_cast<int>(item - static_cast<long long>(z) * per_class);
      tile_n = rest / p.tiles_m;
      tile_m = rest - tile_n * p.tiles_m;
    }
    const int n0 = tile_n * p.bn;
    StrideClass sc{};
    GatherGeom gg;
    int rows_total = p.rows_total, pix_per_img = P, row_pix = p.OW;
    if (mode == 1) {
      sc = stride_class(p, z);
      rows_total = p.K * sc.ra * sc.sb;
      pix_per_img = sc.ha * sc.wb;
      row_pix = sc.wb;
      gg = GatherGeom{P, p.OW, p.OH, p.OW, -1, sc.ra, sc.sb};
    } else {
      gg = GatherGeom{HW, p.W, p.H, p.W, 1, p.R, p.S};
    }
    const long long m_total = static_cast<long long>(p.N) * pix_per_img;
    const long long m0 = static_cast<long long>(tile_m) * 128;
    if (mode != 2 && (m0 >= m_total || rows_total == 0)) continue;   // this class has fewer tiles (or no taps: dx was zeroed by the host)
    const int num_kb = mode == 2 ? p.kb_per_split : (rows_total + 63) / 64;
    const int taps_per_plane = gg.tr * gg.ts;

    // fprop / dgrad: this thread always gathers the same 8 consecutive pixels (chunk `tid & 15` of the
    // 128-pixel tile), for the rows `tid >> 4`, +16, +32, +48 of every reduction block.
    Pix fixed[8];
    Chunk<T> chunk8{};
    TapCursor cur{}, stride_taps{};
    const int step = mode == 1 ? 1 : p.sw;   // distance between the source columns of neighbouring pixels
    if (FAST) {
      stride_taps = tap_cursor(mode == 2 ? kConvThreads / 8 : 16, gg);
      cur = tap_cursor(mode == 2 ? n0 + (tid >> 3) : (tid >> 4), gg);
    }
    if (FAST && mode != 2) {
      const int mfirst = static_cast<int>(m0) + (tid & 15) * 8;
      const int img = mfirst / pix_per_img, rem = mfirst - img * pix_per_img;
      const int py = rem / row_pix, px = rem - py * row_pix;
      const int y0 = mode == 0 ? py * p.sh - p.ph : py + sc.qa;
      const int x0 = mode == 0 ? px * p.sw - p.pw : px + sc.qb;
      const int off0 = mode == 0 ? img * p.C * HW + y0 * p.W + x0 : img * p.K * P + y0 * p.OW + x0;
      chunk8 = make_chunk<T>(src, mfirst < m_total, off0, y0, x0, step, gg);
    }
    if (!FAST && mode != 2) {
      const int mfirst = static_cast<int>(m0) + (tid & 15) * 8;   // the host admits only problems whose pixel counts fit an int
      int img = mfirst / pix_per_img;
      int rem = mfirst - img * pix_per_img;
      int py = rem / row_pix, px = rem - py * row_pix;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (mfirst + e < m_total) {
          if (mode == 0) {
            const int y = py * p.sh - p.ph, x = px * p.sw - p.pw;
            fixed[e] = Pix{img * p.C * HW + y * p.W + x, y, x};
          } else {
            const int y = py + sc.qa, x = px + sc.qb;   // output row / column reached by the tap (ra0, sb0)
            fixed[e] = Pix{img * p.K * P + y * p.OW + x, y, x};
          }
        } else {
          fixed[e] = Pix{0, kNoPixel, kNoPixel};
        }
        if (++px == row_pix) { px = 0; if (++py * row_pix == pix_per_img) { py = 0; ++img; } }
      }
    }

    for (int kb = 0; kb < num_kb && ok; ++kb) {
      if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.err, kErrConvWait)) { ok = false; break; }
      uint8_t* gat = smem + stage * p.stage_bytes;
      uint8_t* tma = gat + p.gather_bytes;
      if (tid == 128) {
        // The operand that needs no gathering: weights (fprop, dgrad) or the output gradient (wgrad).
        if (mode != 2) {
          mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(p.bn) * 128u);
          tma_load_3d(tma, &map_t, &full_bar[stage], kb * 64, n0, z);
        } else {
          const int gkb = split * p.kb_per_split + kb;             // global 64-pixel block: image and offset inside it
          const int img = gkb / kb_img, off = (gkb - img * kb_img) * 64;
          mbar_expect_tx(&full_bar[stage], 128u * 128u);
          tma_load_3d(tma, &map_t, &full_bar[stage], off, 0, img < p.N ? img : p.N);  // an image index past the end reads zeros
        }
      }
      if (mode != 2) {
        // 64 rows (reduction taps) x 128 pixels: two 64-pixel halves of 8 KB each.
        const int chunk = tid & 15, half = chunk >> 3, c16 = chunk & 7;
        if (FAST) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = (tid >> 4) + 16 * j;
            const uint4 v = gather_row<T>(chunk8, cur, cur.tap < rows_total, step, gg);
            advance(cur, stride_taps, gg);
            *reinterpret_cast<uint4*>(gat + half * 8192 + row * 128 + ((c16 ^ (row & 7)) << 4)) = v;
          }
        }
#pragma unroll
        for (int j = 0; j < (FAST ? 0 : 4); ++j) {
          const int row = (tid >> 4) + 16 * j;
          const int tap = kb * 64 + row;
          Pack<T> pk;
          if (tap < rows_total) {
            const int a = tap / taps_per_plane, t2 = tap - a * taps_per_plane, ti = t2 / gg.ts, tj = t2 - ti * gg.ts;
            const int dy = gg.sign * ti, dx = gg.sign * tj;
            const int base = a * gg.plane + dy * gg.rowlen + dx;
#pragma unroll
            for (int e = 0; e < 8; ++e) pk.v[e] = gather_one<T>(src, gg, fixed[e], base, dy, dx);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) pk.v[e] = from_f<T>(0.f);
          }
          *reinterpret_cast<uint4*>(gat + half * 8192 + row * 128 + ((c16 ^ (row & 7)) << 4)) = *reinterpret_cast<uint4*>(&pk);
        }
      } else {
        // bn rows ((c,r,s) taps, the last real one being the column of ones) x 64 pixels of this block.
        const int gkb = split * p.kb_per_split + kb;
        const int img = gkb / kb_img, off = (gkb - img * kb_img) * 64;
        const int c16 = tid & 7;
        if (FAST) {
          const int first = off + c16 * 8;
          const int oh = first / p.OW, ow = first - oh * p.OW;
          const int y0 = oh * p.sh - p.ph, x0 = ow * p.sw - p.pw;
          const bool exists = img < p.N && first < P;
          const Chunk<T> ch = make_chunk<T>(src, exists, img * p.C * HW + y0 * p.W + x0, y0, x0, step, gg);
          const uint32_t one2 = std::is_same<T, __nv_bfloat16>::value ? 0x3f803f80u : 0x3c003c00u;
          TapCursor c = cur;
#pragma unroll 2
          for (int row = tid >> 3; row < p.bn; row += kConvThreads / 8) {
            uint4 v;
            if (c.tap == rows_total - 1) {   // the column of ones: its product with the output gradient is the bias gradient
              const uint32_t o = exists ? one2 : 0u;
              v = make_uint4(o, o, o, o);
            } else {
              v = gather_row<T>(ch, c, c.tap < rows_total - 1, step, gg);
            }
            advance(c, stride_taps, gg);
            *reinterpret_cast<uint4*>(gat + row * 128 + ((c16 ^ (row & 7)) << 4)) = v;
          }
        }
        Pix px[8];
        if (!FAST) {
          const int first = off + c16 * 8;
          int oh = first / p.OW, ow = first - oh * p.OW;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (img < p.N && first + e < P) {
              const int y = oh * p.sh - p.ph, x = ow * p.sw - p.pw;
              px[e] = Pix{img * p.C * HW + y * p.W + x, y, x};
            } else {
              px[e] = Pix{0, kNoPixel, kNoPixel};
            }
            if (++ow == p.OW) { ow = 0; ++oh; }
          }
        }
#pragma unroll 1
        for (int row = tid >> 3; row < (FAST ? 0 : p.bn); row += kConvThreads / 8) {
          const int tap = n0 + row;
          Pack<T> pk;
          if (tap < rows_total - 1) {
            const int c = tap / taps_per_plane, t2 = tap - c * taps_per_plane, r = t2 / p.S, s = t2 - r * p.S;
            const int base = c * HW + r * p.W + s;
#pragma unroll
            for (int e = 0; e < 8; ++e) pk.v[e] = gather_one<T>(src, gg, px[e], base, r, s);
          } else {
            const bool ones = tap == rows_total - 1;   // sums the output gradient: the bias gradient
#pragma unroll
            for (int e = 0; e < 8; ++e) pk.v[e] = from_f<T>((ones && px[e].y != kNoPixel) ? 1.f : 0.f);
          }
          *reinterpret_cast<uint4*>(gat + row * 128 + ((c16 ^ (row & 7)) << 4)) = *reinterpret_cast<uint4*>(&pk);
        }
      }
      fence_async_smem();
      mbar_arrive(&full_bar[stage]);
      if (tid == 128) {
        if (!mbar_wait(&full_bar[stage], phase, p.err, kErrConvWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ga = smem_u32(gat), ta = smem_u32(tma);
        // Reduction rows past the end of the problem are zeros: whole 16-row steps of them are skipped.
        const int ksteps = mode == 2 ? 4 : min(4, (rows_total - kb * 64 + 15) / 16);
        for (int k = 0; k < ksteps; ++k) {
          const uint64_t da = mode != 2 ? make_desc(ga + k * 2048, 8192, 1024) : make_desc(ta + k * 32, 16, 1024);
          const uint64_t db = mode != 2 ? make_desc(ta + k * 32, 16, 1024) : make_desc(ga + k * 32, 16, 1024);
          umma_f16(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (kb == num_kb - 1) umma_commit(done_bar);
      }
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }

    // ---- epilogue: warps 0-3 own the four TMEM lane quarters
    if (warp < 4 && ok) {
      if (mbar_wait(done_bar, tile_count & 1, p.err, kErrConvWait)) {
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        if (mode != 2) {
          const long long m = m0 + warp * 32 + lane;
          const bool live = m < m_total;
          const int img = live ? static_cast<int>(m / pix_per_img) : 0;
          const int rem = live ? static_cast<int>(m - static_cast<long long>(img) * pix_per_img) : 0;
          const int chans = mode == 0 ? p.K : p.C;
          int64_t plane, first;
          if (mode == 0) {
            plane = P;
            first = static_cast<int64_t>(img) * chans * P + rem;
          } else {
            const int i = rem / sc.wb, j = rem - i * sc.wb;
            plane = HW;
            first = static_cast<int64_t>(img) * chans * HW + static_cast<int64_t>(sc.a + p.sh * i) * p.W + sc.b + p.sw * j;
          }
          T* out = static_cast<T*>(p.out) + first;
          const T* bias = static_cast<const T*>(p.bias);
          for (int c0 = 0; c0 < p.bn; c0 += 32) {
            float v[32];
            tmem_ld32(taddr + c0, v);
            if (live) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int ch = n0 + c0 + j;
                if (ch < chans && c0 + j < p.bn) out[static_cast<int64_t>(ch) * plane] = from_f<T>(v[j] + (bias ? to_f(bias[ch]) : 0.f));
              }
            }
          }
        } else {
          const int krow = warp * 32 + lane;   // output channel
          float* out = static_cast<float*>(p.out) + (static_cast<int64_t>(split) * 128 + krow) * p.ldp + n0;
          for (int c0 = 0; c0 < p.bn; c0 += 32) {
            float v[32];
            tmem_ld32(taddr + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (krow < p.K && c0 + j < p.bn) out[c0 + j] = v[j];
          }
        }
      } else {
        ok = false;
      }
    }
    ++tile_count;
    // The next item's first MMA overwrites the accumulator: every epilogue warp must be done reading it.
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, p.tmem_cols);
}

// wgrad second pass: dw[k, tap] and db[k] from the float32 partials.  A block owns 32 consecutive
// outputs; its 8 warps each add every 8th slice in index order and the 8 sums are added in warp
// order, so the result does not depend on scheduling.
template <class T>
__global__ void __launch_bounds__(256) conv_wgrad_finish_kernel(const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db,
                                                                int splits, int K, int CRS, int ldp) {
  __shared__ float part[8][32];
  const int total = K * (CRS + 1);
  const int i = blockIdx.x * 32 + (threadIdx.x & 31), g = threadIdx.x >> 5;
  const int k = i < total ? i / (CRS + 1) : 0, tap = i < total ? i - k * (CRS + 1) : 0;
  float acc = 0.f;
  if (i < total)
    for (int s = g; s < splits; s += 8) acc += partial[(static_cast<int64_t>(s) * 128 + k) * ldp + tap];
  part[g][threadIdx.x & 31] = acc;
  __syncthreads();
  if (g == 0 && i < total) {
    float sum = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) sum += part[q][threadIdx.x];
    if (tap < CRS) dw[static_cast<int64_t>(k) * CRS + tap] = from_f<T>(sum);
    else if (db != nullptr) db[k] = from_f<T>(sum);
  }
}

// Weights for the input gradient, one matrix per stride class z = a * sw + b:
//   wt[z][c][(k, ri, si)] = w[k][c][ra0 + ri*sh][sb0 + si*sw]   (the taps that class can see),
// rows padded with zeros to `ld` elements.
template <class T>
__global__ void conv_permute_weight_kernel(const T* __restrict__ w, T* __restrict__ wt, ConvParams p, int ld) {
  const int total = p.classes * p.C * ld;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int z = i / (p.C * ld), rest = i - z * (p.C * ld), c = rest / ld, q = rest - c * ld;
    const StrideClass sc = stride_class(p, z);
    const int taps = sc.ra * sc.sb;
    T v = from_f<T>(0.f);
    if (q < p.K * taps) {
      const int k = q / taps, t = q - k * taps, ri = t / sc.sb, si = t - ri * sc.sb;
      v = w[((static_cast<int64_t>(k) * p.C + c) * p.R + sc.ra0 + ri * p.sh) * p.S + sc.sb0 + si * p.sw];
    }
    wt[i] = v;
  }
}
template <class T>
__global__ void conv_pad_rows_kernel(const T* __restrict__ w, T* __restrict__ wp, int rows, int cols, int ld) {
  const int total = rows * ld;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int r = i / ld, q = i - r * ld;
    wp[i] = q < cols ? w[static_cast<int64_t>(r) * cols + q] : from_f<T>(0.f);
  }
}

ConvGeometry geometry_of(const Shape& x, const Shape& w, const int64_t* i) {
  ConvGeometry g;
  g.N = static_cast<int>(x[0]); g.C = static_cast<int>(x[1]); g.H = static_cast<int>(x[2]); g.W = static_cast<int>(x[3]);
  g.K = static_cast<int>(w[0]); g.R = static_cast<int>(w[2]); g.S = static_cast<int>(w[3]);
  g.sh = static_cast<int>(i[0]); g.sw = static_cast<int>(i[1]); g.ph = static_cast<int>(i[2]); g.pw = static_cast<int>(i[3]);
  return g;
}

// Kernel arguments from the plan (pointers are filled in by the caller).
ConvParams params_of(const ConvGeometry& g, const ConvPlan& plan, int device) {
  ConvParams p{};
  p.mode = static_cast<int>(plan.pass);
  p.N = g.N; p.C = g.C; p.H = g.H; p.W = g.W; p.K = g.K; p.R = g.R; p.S = g.S;
  p.OH = plan.out_h; p.OW = plan.out_w; p.sh = g.sh; p.sw = g.sw; p.ph = g.ph; p.pw = g.pw;
  p.rows_total = plan.rows_total; p.bn = plan.bn; p.tiles_m = plan.tiles_m; p.tiles_n = plan.tiles_n;
  p.classes = plan.classes; p.splits = plan.splits; p.kb_per_split = plan.kb_per_split; p.ldp = plan.ldp;
  p.gather_bytes = plan.gather_bytes; p.stage_bytes = plan.stage_bytes; p.stages = plan.stages; p.tmem_cols = plan.tmem_cols;
  p.err = tc05_error_flag(device);
  return p;
}

bool route_allowed(const Tensor& t) {
  const char* env = std::getenv("ORTHON_CUDA_CONV2D");
  if (env && (std::strcmp(env, "direct") == 0 || std::strcmp(env, "gemm") == 0)) return false;
  if (t.dtype() != DType::BF16 && t.dtype() != DType::F16) return false;
  return Runtime::instance().cuda(t.device().index).supports_tcgen05();
}

int g_last_launch[4] = {0, 0, 0, 0};   // grid, dynamic shared memory, ring slots, CTAs per SM of the latest launch (diagnostics)

// A persistent grid: as many CTAs as can be resident, each walking the work items with a stride of the grid.
template <class T, int MODE, bool FAST>
void launch_mode(const CUtensorMap& map, const ConvParams& p, const ConvPlan& plan, cudaStream_t st) {
  // The largest shared-memory carve-out, or a CTA that needs under half of it gets an SM configured for one CTA only.
  static const bool once = (cudaFuncSetAttribute(conv_tc05_kernel<T, MODE, FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, kConvSmemMax),
                            prefer_max_shared_carveout(conv_tc05_kernel<T, MODE, FAST>), true);
  (void)once;
  g_last_launch[0] = plan.grid; g_last_launch[1] = plan.smem_bytes; g_last_launch[2] = plan.stages; g_last_launch[3] = plan.ctas_per_sm;
  conv_tc05_kernel<T, MODE, FAST><<<static_cast<unsigned>(plan.grid), kConvThreads, plan.smem_bytes, st>>>(map, p);
}

template <class T>
void launch(const CUtensorMap& map, const ConvParams& p, const ConvPlan& plan, cudaStream_t st) {
  const bool fast = plan.fast;
  if (p.mode == 0) fast ? launch_mode<T, 0, true>(map, p, plan, st) : launch_mode<T, 0, false>(map, p, plan, st);
  else if (p.mode == 1) fast ? launch_mode<T, 1, true>(map, p, plan, st) : launch_mode<T, 1, false>(map, p, plan, st);
  else fast ? launch_mode<T, 2, true>(map, p, plan, st) : launch_mode<T, 2, false>(map, p, plan, st);
}

// Tensor map over `mats` row-major [rows, ld] matrices of 16-bit elements laid one after another:
// a rank-3 map (inner, rows, mats).
bool matrix_map(CUtensorMap* out, DType dt, void* base, int inner, int rows, int mats, int ld, int box_rows) {
  const uint64_t dims[3] = {static_cast<uint64_t>(inner), static_cast<uint64_t>(rows), static_cast<uint64_t>(mats)};
  const uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(rows)};
  const uint32_t box[3] = {64, static_cast<uint32_t>(box_rows), 1};
  return tc05_encode_map(out, dt, 3, base, dims, strides, box);
}

}  // namespace

// {grid, dynamic shared memory bytes, ring slots, resident CTAs per SM} of the latest implicit-GEMM launch.
std::vector<int> conv_tc05_last_launch() { return std::vector<int>(g_last_launch, g_last_launch + 4); }

template <class T>
bool conv_fprop_tc05(OpCall& c) {
  const Tensor &x = c.in[0], &w = c.in[1];
  if (!route_allowed(x)) return false;
  const ConvGeometry g = geometry_of(x.shape(), w.shape(), c.i);
  const int sms = sm_count_for(x);
  const ConvPlan plan = plan_conv(ConvPass::Forward, g, sms);
  if (!plan.eligible) return false;
  cudaStream_t st = stream_of(c);
  // The TMA row pitch must be a multiple of 16 bytes: weights whose rows are not get a padded copy.
  Tensor wp = w;
  if (plan.pad_weights) {
    wp = Tensor::empty({g.K, plan.weight_ld}, w.dtype(), w.device());
    conv_pad_rows_kernel<T><<<ew_grid(wp.numel(), 256, sms), 256, 0, st>>>(w.data_as<T>(), wp.data_as<T>(), g.K, plan.rows_total, plan.weight_ld);
  }
  ConvParams p = params_of(g, plan, x.device().index);
  p.src = x.data(); p.out = c.out[0].data(); p.bias = c.in[2].defined() ? c.in[2].data() : nullptr;
  CUtensorMap map;
  if (!matrix_map(&map, w.dtype(), const_cast<void*>(wp.data()), plan.weight_ld, g.K, 1, plan.weight_ld, plan.bn)) return false;
  launch<T>(map, p, plan, st);
  check_launch("conv2d (implicit GEMM)");
  return true;
}

template <class T>
bool conv_dgrad_tc05(OpCall& c) {
  const Tensor &gy = c.in[0], &w = c.in[1];
  Tensor& dx = c.out[0];
  if (!route_allowed(gy)) return false;
  const ConvGeometry g = geometry_of(dx.shape(), w.shape(), c.i);
  const int sms = sm_count_for(gy);
  const ConvPlan plan = plan_conv(ConvPass::InputGradient, g, sms);
  if (!plan.eligible) return false;
  cudaStream_t st = stream_of(c);
  ConvParams p = params_of(g, plan, gy.device().index);
  Tensor wt = Tensor::empty({plan.classes, g.C, plan.weight_ld}, w.dtype(), w.device());
  conv_permute_weight_kernel<T><<<ew_grid(wt.numel(), 256, sms), 256, 0, st>>>(w.data_as<T>(), wt.data_as<T>(), p, plan.weight_ld);
  // A stride larger than the filter leaves input pixels that no tap reaches: their gradient is zero.
  if (plan.zero_fill) OB_CUDA(cudaMemsetAsync(dx.data(), 0, dx.nbytes(), st));
  p.src = gy.data(); p.out = dx.data(); p.bias = nullptr;
  CUtensorMap map;
  if (!matrix_map(&map, w.dtype(), wt.data(), plan.weight_ld, g.C, plan.classes, plan.weight_ld, plan.bn)) return false;
  launch<T>(map, p, plan, st);
  check_launch("conv2d input gradient (implicit GEMM)");
  return true;
}

// Also produces the bias gradient (c.out[1], when defined) from the column of ones and reports
// that through c.i[4] = 1.
template <class T>
bool conv_wgrad_tc05(OpCall& c) {
  const Tensor &gy = c.in[0], &x = c.in[1];
  Tensor& dw = c.out[0];
  if (!route_allowed(gy)) return false;
  const ConvGeometry g = geometry_of(x.shape(), dw.shape(), c.i);
  const int sms = sm_count_for(gy);
  const ConvPlan plan = plan_conv(ConvPass::WeightGradient, g, sms);
  if (!plan.eligible) return false;
  cudaStream_t st = stream_of(c);
  ConvParams p = params_of(g, plan, gy.device().index);
  const int P = plan.out_h * plan.out_w, CRS = plan.rows_total - 1;
  Tensor partial = Tensor::empty({plan.splits, 128, plan.ldp}, DType::F32, gy.device());
  p.src = x.data(); p.out = partial.data(); p.bias = nullptr;
  // gy as [N][K][P]: inner = pixel, rows = channel, outer = image; rows past K and images past N read zeros.
  CUtensorMap map;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(P), static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.N)};
    const uint64_t strides[2] = {static_cast<uint64_t>(P) * 2, static_cast<uint64_t>(P) * 2 * static_cast<uint64_t>(g.K)};
    const uint32_t box[3] = {64, 128, 1};
    if (!tc05_encode_map(&map, gy.dtype(), 3, const_cast<void*>(gy.data()), dims, strides, box)) return false;
  }
  launch<T>(map, p, plan, st);
  T* db = c.out[1].defined() ? c.out[1].data_as<T>() : nullptr;
  conv_wgrad_finish_kernel<T><<<static_cast<unsigned>((static_cast<int64_t>(g.K) * plan.rows_total + 31) / 32), 256, 0, st>>>(
      partial.data_as<float>(), dw.data_as<T>(), db, plan.splits, g.K, CRS, plan.ldp);
  if (db != nullptr) c.i[4] = 1;
  check_launch("conv2d weight gradient (implicit GEMM)");
  return true;
}

template bool conv_fprop_tc05<__nv_bfloat16>(OpCall&);
template bool conv_fprop_tc05<__half>(OpCall&);
template bool conv_dgrad_tc05<__nv_bfloat16>(OpCall&);
template bool conv_dgrad_tc05<__half>(OpCall&);
template bool conv_wgrad_tc05<__nv_bfloat16>(OpCall&);
template bool conv_wgrad_tc05<__half>(OpCall&);

}  // namespace cu
}  // namespace ob

// gemm_tc05: bf16 / fp16 GEMM on the 5th-generation tensor cores (sm_100a).
//
//   D[b] = epilogue( op(A[b]) @ op(B[b]) )        fp32 accumulation in tensor memory
//
// Design
//  * Persistent kernel, one CTA per SM, tiles of 128 x BN (BN = 256 or 128) x 64.
//  * Warp-specialised: warp 0 issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, every
//    CTA fetches its own tiles) into a multi-stage shared-memory ring guarded by mbarriers; warp 1
//    issues tcgen05.mma (one elected thread) with the accumulator in TMEM and releases ring
//    slots with tcgen05.commit; warps 2-5 drain the accumulator with tcgen05.ld and run the
//    fused epilogue (bias, ReLU/GELU, residual add, optional pre-activation copy, dtype
//    conversion); rows are staged in swizzled shared memory and leave as TMA stores of full
//    128-byte lines.  Two TMEM accumulators (2 x BN columns) let the epilogue of tile i overlap
//    the main loop of tile i+1.  The epilogue is one rolled loop over 32-column slices so that
//    the whole kernel body stays inside the instruction cache.
//  * Both operands may be K-major or MN-major: transposed operands (the backward GEMMs) are
//    described by shared-memory descriptors instead of being packed, and up to two batch
//    dimensions with arbitrary strides go through rank-4 tensor maps, so attention heads are
//    read in place from a packed QKV activation.
//  * Every mbarrier wait is bounded by a clock budget; on expiry the kernel raises an error
//    word and unwinds (TMEM is always released), so a logic error can never hang the GPU.
//
// A SIMT kernel handles float32 (exact, for parity tests) and operands that violate TMA
// alignment rules.
//
// Replaces (reference project paths): src/backends/cuda/matmul_kernels.cu:51-134 (cuBLAS
// routes), :138-400 (16x16 SIMT tiles), src/backends/cuda/fusion_kernels.cu:42-86.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "ob/cuda_common.cuh"
#include "ob/gemm_plan.h"
#include "ob/ops.h"
#include "ob/tc05.cuh"

namespace ob {
namespace cu {

void strided_copy_cuda(const Tensor& src, Tensor& dst, cudaStream_t st);

namespace {

using namespace tc05;

// Planner options: the environment's values, read once, plus the settings that bindings can
// change at run time (forced route for diagnostics, float32 precision, CTA-pair mode).
std::atomic<int> g_force_route{0};     // 0 = planner decides, 1 = force the SIMT kernel, 2 = require tcgen05
std::atomic<int> g_last_route{0};      // GemmRoute of the last product
std::atomic<int> g_last_plan_bn{0};    // tile width of the last product
std::atomic<int> g_f32_precision{-1};  // -1 = as the environment says
std::atomic<int> g_pair_mode{-2};      // -2 = as the environment says
GemmPlanOptions plan_options() {
  static const GemmPlanOptions from_env = GemmPlanOptions::from_environment();
  GemmPlanOptions o = from_env;
  o.force_route = g_force_route.load(std::memory_order_relaxed);
  const int f32 = g_f32_precision.load(std::memory_order_relaxed);
  if (f32 >= 0) o.float32_precision = f32;
  const int pair = g_pair_mode.load(std::memory_order_relaxed);
  if (pair != -2) o.pair_mode = pair;
  return o;
}
int f32_precision() { return plan_options().float32_precision; }

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpilogueWarps = 4;
// TMA warp, MMA warp, four epilogue warps per MMA row block of the tile.
constexpr int gemm_threads(int tile_rows, int epilogue_warps = kEpilogueWarps) { return 32 * (2 + epilogue_warps * (tile_rows / 128)); }

enum : int { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3 };

struct GemmParams {
  int M, N, K;
  int nb0, nb1;                 // batch extents (outer, inner)
  int a_mn, b_mn;               // operand majors (0 = K-major, 1 = MN-major)
  int a_bc, b_bc;               // 1 = operand is shared by every batch entry (batch stride 0)
  int bias_rows;                // 1 = bias is indexed by output row instead of column
  int tma_store;                // 1 = epilogue stages tiles in shared memory and stores them with TMA
  int out_f32;                  // 1 = C and bias are float32 (operands are bfloat16 pieces of float32 values)
  void* C; long long ldc, c_bs0, c_bs1;
  const void* bias;             // [N] or null
  const void* residual; long long ldr, r_bs0, r_bs1;
  void* preact;                 // same layout as C, or null
  int act;                      // 0 none, 1 relu, 2 gelu
  int* err;
};

// TM = rows of the CTA tile: 128 (one MMA row block, accumulators double-buffered across tiles) or
// 256 (two MMA row blocks share every B stage, which halves the B bytes fetched per flop; the two
// accumulators are drained one after the other so the next tile can start on the first).
// PAIR: the tile belongs to a pair of CTAs (cta_group::2): TM rows of A and BN / 2 columns of B
// per CTA, 2 TM x BN outputs per pair.
template <int BN, int TM, bool PAIR = false>
struct SmemLayout {
  static constexpr int kABytes = TM * BK * 2;
  static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiBytes = kEpilogueWarps * 2 * 4096;  // two 32x64 staging tiles per epilogue warp
  static constexpr int kStages = (232448 - kEpiBytes - 256 - 1024) / kStageBytes > 6 ? 6 : (232448 - kEpiBytes - 256 - 1024) / kStageBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kEpiBytes + kBarrierBytes + 1024;  // +1024 for manual alignment
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return v > 0.f ? v : 0.f;
  if (act == 2) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}

// d/dz of 0.5 z (1 + erf(z / sqrt 2)).
__device__ __forceinline__ float gelu_grad(float z) {
  return 0.5f * (1.f + erff(z * 0.70710678118654752f)) + z * 0.3989422804014327f * __expf(-0.5f * z * z);
}

// EW = epilogue warps per MMA row block: 4, or 8 for 128-row tiles with short reductions, where
// draining a 128 x 256 accumulator takes longer than computing the next one: two warps then share
// each TMEM lane quarter and take half of the columns each.
//
// PAIR = true is the two-CTA form (launched as clusters of two, TM = 128, BN = 256): the pair
// computes a 256 x 256 tile with tcgen05.mma.cta_group::2.  CTA r of the pair loads rows
// [r * 128, r * 128 + 128) of the A tile and columns [r * 128, r * 128 + 128) of the B tile (its
// own non-multicast TMA loads, completion counted on the even CTA's barrier), holds the
// accumulator rows of its A half in its own tensor memory (two 256-column accumulators, so the
// epilogue of a tile overlaps the main loop of the next) and stores its own output rows.  The
// even CTA issues every MMA and commits to both CTAs' barriers; each SM's tensor core reads 32 KB
// of shared memory per 128 x 256 x 64 block instead of 48 KB, which is what a power-capped GPU
// converts into clock.
template <class T, int BN, int TM, int EW = kEpilogueWarps, bool PAIR = false>
__global__ void __launch_bounds__(gemm_threads(TM, EW), 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_z, GemmParams p) {
  using L = SmemLayout<BN, TM, PAIR>;
  constexpr int H = TM / BM;  // MMA row blocks per tile
  static_assert(EW == 4 || (EW == 8 && H == 1 && BN == 256), "eight epilogue warps are for the 128 x 256 tile");
  static_assert(!PAIR || BN == 256, "the pair form is a (2 TM) x 256 tile over two CTAs");
  constexpr int TILE_M = PAIR ? 2 * TM : TM;        // rows of the scheduling tile
  constexpr int BNC = PAIR ? BN / 2 : BN;           // B columns this CTA loads
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0;
  const long long first_tile = PAIR ? blockIdx.x / 2 : blockIdx.x;
  const long long tile_step = PAIR ? gridDim.x / 2 : gridDim.x;
  constexpr bool kSplitCols = EW == 8;        // two warps per lane quarter, half of the columns each
  constexpr bool kOneStage = H == 2 || EW == 8;  // one 4 KB staging tile per epilogue warp
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + L::kStages * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_smem + L::kEpiBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* tmem_full = empty_bar + L::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + TILE_M - 1) / TILE_M, tiles_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = tiles_m * tiles_n;
  const long long total_tiles = static_cast<long long>(tiles_per_batch) * p.nb0 * p.nb1;
  const int num_kb = (p.K + BK - 1) / BK;
  // Accumulator slot and use count of row block h of this CTA's it-th tile.
  auto slot_of = [](int it, int h) { return H == 1 ? (it & 1) : h; };
  auto use_of = [](int it) { return H == 1 ? (it >> 1) : it; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], PAIR ? 2 * EW : EW); }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tile order: groups of 8 M-tiles sweep N together so concurrently resident CTAs share
  // operand panels in L2.
  auto decode_tile = [&](long long t, int& bidx, int& tm, int& tn) {
    bidx = static_cast<int>(t / tiles_per_batch);
    const int r = static_cast<int>(t - static_cast<long long>(bidx) * tiles_per_batch);
    constexpr int G = 8;
    const int group = r / (G * tiles_n);
    const int first_m = group * G;
    const int gsize = min(G, tiles_m - first_m);
    const int in_group = r - group * G * tiles_n;
    tm = first_m + in_group % gsize;
    tn = in_group / gsize;
  };

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Pair form: the bytes of both CTAs are counted on the even CTA's barrier of the stage.
      const uint32_t pair_full0 = PAIR ? mapa_u32(smem_u32(&full_bar[0]), 0u) : 0u;
      for (long long t = first_tile; t < total_tiles && ok; t += tile_step) {
        int bidx, tm, tn;
        decode_tile(t, bidx, tm, tn);
        const int b0 = bidx / p.nb1, b1 = bidx - b0 * p.nb1;
        const int a0 = p.a_bc ? 0 : b0, a1 = p.a_bc ? 0 : b1, c0 = p.b_bc ? 0 : b0, c1 = p.b_bc ? 0 : b1;
        const int row_a = tm * TILE_M + static_cast<int>(crank) * TM, col_b = tn * BN + static_cast<int>(crank) * BNC;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.err, kErrProducer)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full_bar[stage], PAIR ? 2 * L::kStageBytes : L::kStageBytes);
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const int k0 = kb * BK;
          const uint32_t pair_full = pair_full0 + stage * 8;
          auto load = [&](uint8_t* dst, const CUtensorMap* map, int x, int y, int z, int w) {
            if (PAIR) tma_load_4d_pair(dst, map, pair_full, x, y, z, w);
            else tma_load_4d(dst, map, &full_bar[stage], x, y, z, w);
          };
          if (!p.a_mn) {
            load(sa, &map_a, k0, row_a, a1, a0);
          } else {
#pragma unroll
            for (int c = 0; c < TM / 64; ++c) load(sa + c * (BK * 128), &map_a, row_a + c * 64, k0, a1, a0);
          }
          if (!p.b_mn) {
            load(sb, &map_b, k0, col_b, c1, c0);
          } else {
#pragma unroll
            for (int c = 0; c < BNC / 64; ++c) load(sb + c * (BK * 128), &map_b, col_b + c * 64, k0, c1, c0);
          }
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    if (lane == 0 && leader) {
      // Instruction descriptor: fp32 accumulate, A/B format, majors, N>>3, M>>4 (256 rows for a pair).
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(p.a_mn) << 15) |
                             (static_cast<uint32_t>(p.b_mn) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>((PAIR ? 2 * BM : BM) >> 4) << 24);
      // Pair form: every commit goes to this CTA's barrier and to the peer's.
      const uint32_t peer_empty0 = PAIR ? mapa_u32(smem_u32(&empty_bar[0]), 1u) : 0u;
      const uint32_t peer_tmem_full0 = PAIR ? mapa_u32(smem_u32(&tmem_full[0]), 1u) : 0u;
      // Descriptors are built once; every other one is this plus an offset in 16-byte units (the
      // issuing thread has about 500 tensor cycles per 64-wide K block to spend, and rebuilding
      // eight descriptors per block used most of them).
      const uint64_t da0 = p.a_mn ? make_desc(smem_u32(smem), BK * 128, 1024) : make_desc(smem_u32(smem), 16, 1024);
      const uint64_t db0 = p.b_mn ? make_desc(smem_u32(smem) + L::kABytes, BK * 128, 1024) : make_desc(smem_u32(smem) + L::kABytes, 16, 1024);
      const uint32_t a_step = p.a_mn ? 2048u >> 4 : 32u >> 4, b_step = p.b_mn ? 2048u >> 4 : 32u >> 4;  // one K = 16 slice
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (long long t = first_tile; t < total_tiles && ok; t += tile_step, ++it) {
        const uint32_t empty_parity = (use_of(it) & 1) ^ 1;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.err, kErrMma)) { ok = false; break; }
          tc_fence_after();
          if (kb == 0) {  // the accumulators must have been drained by the epilogue
#pragma unroll
            for (int h = 0; h < H; ++h)
              if (ok && !mbar_wait(&tmem_empty[slot_of(it, h)], empty_parity, p.err, kErrMma)) ok = false;
            if (!ok) break;
            tc_fence_after();
          }
          const uint64_t da_s = da0 + static_cast<uint32_t>(stage * (L::kStageBytes >> 4));
          const uint64_t db_s = db0 + static_cast<uint32_t>(stage * (L::kStageBytes >> 4));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t db = db_s + k * b_step;
#pragma unroll
            for (int h = 0; h < H; ++h) {
              const uint64_t da = da_s + k * a_step + h * ((BM * BK * 2) >> 4);  // 128 rows further in either operand major
              if (PAIR) umma_f16_pair(tmem_base + slot_of(it, h) * BN, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
              else umma_f16(tmem_base + slot_of(it, h) * BN, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          // Frees the slot (in both CTAs of a pair) once these MMAs have read it.
          if (PAIR) { umma_commit_pair(smem_u32(&empty_bar[stage])); umma_commit_pair(peer_empty0 + stage * 8); }
          else umma_commit(&empty_bar[stage]);
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
            if (PAIR) { umma_commit_pair(smem_u32(&tmem_full[slot_of(it, h)])); umma_commit_pair(peer_tmem_full0 + slot_of(it, h) * 8); }
            else umma_commit(&tmem_full[slot_of(it, h)]);
          }
        }
      }
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    bool ok = true;
    int it = 0;
    T* Cb = static_cast<T*>(p.C);
    const T* Rb = static_cast<const T*>(p.residual);
    T* Zb = static_cast<T*>(p.preact);
    const T* bias = static_cast<const T*>(p.bias);
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) &&
                        (p.c_bs0 % 8 == 0) && (p.c_bs1 % 8 == 0) &&
                        (!Rb || ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(Rb) & 15u) == 0) && (p.r_bs0 % 8 == 0) && (p.r_bs1 % 8 == 0))) &&
                        (!Zb || ((reinterpret_cast<uintptr_t>(Zb) & 15u) == 0)) &&
                        (!bias || ((reinterpret_cast<uintptr_t>(bias) & 15u) == 0));
    // One loop body for every output mode keeps the epilogue code small enough to stay resident
    // in the instruction cache next to the producer and MMA loops.  Per 32-column slice: load the
    // accumulators, add bias, optionally write the pre-activation, activate, add the residual,
    // write the result.  Writing is either (a) staged: each lane puts its row into a swizzled
    // 32x64 shared-memory tile that one TMA store moves out as full 128-byte lines (edges clipped
    // by the tensor map), or (b) direct 16-byte / scalar stores when the output is not TMA-friendly.
    const bool staged = p.tma_store != 0;
    const bool vec = staged || (vec_ok && (p.N % 8 == 0));
    // Staging: two 4 KB tiles per warp with one row block, one per warp with two (the row blocks
    // are then drained concurrently by their own four warps).
    uint8_t* ebuf = epi_smem + (warp - 2) * (kOneStage ? 4096 : 8192);
    const int my_h = (warp - 2) >> 2;   // row block (H == 2) or column half (EW == 8) of this warp
    constexpr int kSubs = BN / 32;
    const int sub_begin = kSplitCols ? my_h * (kSubs / 2) : 0, sub_end = kSplitCols ? sub_begin + kSubs / 2 : kSubs;
    int buf = 0;
    // One staging tile and two outputs: the second output (stored pre-activation or activation
    // derivative) waits, packed to 16 bits in registers, until the store of the result has read
    // the tile, and then goes out through the same tile.
    const bool defer_z = kOneStage && staged && Zb != nullptr;
    uint4 zp0[4], zp1[4];   // the two 32-column halves of a 64-column group (named, not indexed: they stay in registers)
    // Pair form: the even CTA's MMA thread waits for the epilogue warps of both CTAs.
    const uint32_t pair_tmem_empty0 = PAIR ? mapa_u32(smem_u32(&tmem_empty[0]), 0u) : 0u;
    for (long long t = first_tile; t < total_tiles && ok; t += tile_step, ++it) {
      int bidx, tm, tn;
      decode_tile(t, bidx, tm, tn);
      const int b0 = bidx / p.nb1, b1 = bidx - b0 * p.nb1;
#pragma unroll 1
      for (int h = 0; h < H && ok; ++h) {
      if (H == 2 && h != my_h) continue;
      const int acc = slot_of(it, h);
      if (!mbar_wait(&tmem_full[acc], use_of(it) & 1, p.err, kErrEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int row0 = tm * TILE_M + static_cast<int>(crank) * TM + h * BM + quarter * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const long long c_off = b0 * p.c_bs0 + b1 * p.c_bs1 + static_cast<long long>(row) * p.ldc;
      const long long r_off = b0 * p.r_bs0 + b1 * p.r_bs1 + static_cast<long long>(row) * p.ldr;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const float bias_row = (bias && p.bias_rows && row_ok && !p.out_f32) ? to_f(bias[row]) : 0.f;
#pragma unroll 1
      for (int sub = sub_begin; sub < sub_end; ++sub) {
        const int col0 = tn * BN + sub * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        float v[32];
        tmem_ld32(taddr + sub * 32, v);
        if (row0 >= p.M) continue;  // uniform: none of this warp's rows exist
        if (p.out_f32) {
          // Float32 output: bias and activation in float, each lane stores its 32 columns (one
          // 128-byte line) directly.
          const float* bias_f = static_cast<const float*>(p.bias);
          if (bias_f) {
            const float br = (p.bias_rows && row_ok) ? bias_f[row] : 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += p.bias_rows ? br : ((col0 + j < p.N) ? bias_f[col0 + j] : 0.f);
          }
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
          } else if (p.act == 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.5f * v[j] * (1.f + erff(v[j] * 0.70710678118654752f));
          }
          if (row_ok) {
            float* dst = static_cast<float*>(p.C) + c_off + col0;
            if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q) reinterpret_cast<float4*>(dst)[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dst[j] = v[j];
            }
          }
          continue;
        }
        const int half = sub & 1;
        if (staged && half == 0) {
          // The tile about to be overwritten must have been read by its previous store.
          if (lane == 0) {
            if (Zb || kOneStage) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          }
          __syncwarp();
        }
        auto emit = [&](T* base, uint8_t* tile, bool is_z, const float* vals) {
          if (staged) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              Pack<T> pk;
#pragma unroll
              for (int j = 0; j < 8; ++j) pk.v[j] = from_f<T>(vals[q * 8 + j]);
              *reinterpret_cast<uint4*>(tile + lane * 128 + (((half * 4 + q) ^ (lane & 7)) << 4)) = *reinterpret_cast<uint4*>(&pk);
            }
            if (half == 1 || col0 + 32 >= p.N) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                if (is_z) tma_store_4d(&map_z, tile, col0 - half * 32, row0, b1, b0);
                else tma_store_4d(&map_c, tile, col0 - half * 32, row0, b1, b0);
              }
            }
          } else if (row_ok) {
            if (vec) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (col0 + q * 8 < p.N) {
                  Pack<T> pk;
#pragma unroll
                  for (int j = 0; j < 8; ++j) pk.v[j] = from_f<T>(vals[q * 8 + j]);
                  store_pack(base + c_off + col0 + q * 8, pk);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) base[c_off + col0 + j] = from_f<T>(vals[j]);
            }
          }
        };
        if (bias) {
          if (p.bias_rows) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += bias_row;
          } else if (vec) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col0 + q * 8 < p.N) {
                Pack<T> pb = load_pack(bias + col0 + q * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[q * 8 + j] += to_f(pb.v[j]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += to_f(bias[col0 + j]);
          }
        }
        if (p.act == 4) {
          // GELU forward that also returns its derivative (kept for the backward pass in place of
          // the pre-activation): one erf serves both.
          float d[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float cdf = 0.5f * (1.f + erff(v[j] * 0.70710678118654752f));
            d[j] = cdf + v[j] * 0.3989422804014327f * __expf(-0.5f * v[j] * v[j]);
            v[j] *= cdf;
          }
          if (defer_z) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              Pack<T> pk;
#pragma unroll
              for (int j = 0; j < 8; ++j) pk.v[j] = from_f<T>(d[q * 8 + j]);
              if (half == 0) zp0[q] = *reinterpret_cast<uint4*>(&pk);
              else zp1[q] = *reinterpret_cast<uint4*>(&pk);
            }
          } else if (Zb) {
            emit(Zb, ebuf, true, d);
          }
        } else {
          if (defer_z) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              Pack<T> pk;
#pragma unroll
              for (int j = 0; j < 8; ++j) pk.v[j] = from_f<T>(v[q * 8 + j]);
              if (half == 0) zp0[q] = *reinterpret_cast<uint4*>(&pk);
              else zp1[q] = *reinterpret_cast<uint4*>(&pk);
            }
          } else if (Zb) {
            emit(Zb, ebuf, true, v);
          }
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
          } else if (p.act == 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.5f * v[j] * (1.f + erff(v[j] * 0.70710678118654752f));
          }
        }
        if (Rb && row_ok) {
          // act 3: the result is acc * aux (aux = stored activation derivative: the input gradient
          // of a GELU MLP); otherwise aux is a residual that is added.
          float aux[32];
          if (vec) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              Pack<T> pr;
              if (col0 + q * 8 < p.N) pr = load_pack(Rb + r_off + col0 + q * 8);
#pragma unroll
              for (int j = 0; j < 8; ++j) aux[q * 8 + j] = (col0 + q * 8 < p.N) ? to_f(pr.v[j]) : 0.f;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) aux[j] = (col0 + j < p.N) ? to_f(Rb[r_off + col0 + j]) : 0.f;
          }
          if (p.act == 3) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= aux[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += aux[j];
          }
        }
        emit(Cb, kOneStage ? ebuf : (Zb ? ebuf + 4096 : ebuf + buf * 4096), false, v);
        if (!kOneStage && staged && !Zb && (half == 1 || col0 + 32 >= p.N)) buf ^= 1;
        if (defer_z && (half == 1 || col0 + 32 >= p.N)) {
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the result's store has read the tile
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(ebuf + lane * 128 + ((q ^ (lane & 7)) << 4)) = zp0[q];
          if (half == 1) {
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(ebuf + lane * 128 + (((4 + q) ^ (lane & 7)) << 4)) = zp1[q];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) tma_store_4d(&map_z, ebuf, col0 - half * 32, row0, b1, b0);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(pair_tmem_empty0 + acc * 8);
        else mbar_arrive(&tmem_empty[acc]);
      }
      }  // row block
    }
    if (staged) {
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      __syncwarp();
    }
  }

  tc_fence_before();
  __syncthreads();
  // Neither CTA of a pair may leave (or give up its tensor memory) while the other can still
  // arrive on its barriers or while pair MMAs that write both tensor memories are in flight.
  if (PAIR) cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------- SIMT fallback
// 64x64 output tile, 16x16 threads, 4x4 outputs per thread; arbitrary element strides.
template <class T>
__global__ void gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int M, int N, int K,
                                 long long a_sm, long long a_sk, long long b_sk, long long b_sn, long long ldc,
                                 int nb1, long long a_bs0, long long a_bs1, long long b_bs0, long long b_bs1,
                                 long long c_bs0, long long c_bs1, const T* __restrict__ bias, const T* __restrict__ residual,
                                 long long ldr, long long r_bs0, long long r_bs1, T* __restrict__ preact, int act, int bias_rows) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
  A += b0 * a_bs0 + b1 * a_bs1;
  B += b0 * b_bs0 + b1 * b_bs1;
  const long long c_base = b0 * c_bs0 + b1 * c_bs1;
  const long long r_base = b0 * r_bs0 + b1 * r_bs1;
  const int tx = threadIdx.x, ty = threadIdx.y, tid = ty * 16 + tx;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = tid; i < 64 * 16; i += 256) {
      const int kk = i % 16, mm = i / 16;
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? to_f(A[gm * a_sm + gk * a_sk]) : 0.f;
      const int nn = i % 64, kb = i / 64;
      const int gn = n0 + nn, gk2 = k0 + kb;
      Bs[kb][nn] = (gn < N && gk2 < K) ? to_f(B[gk2 * b_sk + gn * b_sn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) {
        float x = acc[i][j];
        if (bias) x += to_f(bias[bias_rows ? gm : gn]);
        if (preact) preact[c_base + gm * ldc + gn] = from_f<T>(act == 4 ? gelu_grad(x) : x);
        x = apply_act(x, act == 4 ? 2 : act);
        if (residual) {
          const float aux = to_f(residual[r_base + gm * ldr + gn]);
          x = (act == 3) ? x * aux : x + aux;
        }
        C[c_base + gm * ldc + gn] = from_f<T>(x);
      }
    }
}

// Large-tile SIMT kernel: 128 x 128 output tile, 16 x 16 threads, 8 x 8 outputs per thread (two
// 4-wide row groups and two 4-wide column groups, so shared-memory reads are conflict-free
// float4 accesses), reduction in steps of 16 with the next step's operands prefetched into
// registers while the current one is multiplied.  Arbitrary element strides; the fast thread
// index follows whichever stride of each operand is 1.
template <class T>
__global__ void __launch_bounds__(256, 1)
gemm_simt128_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int M, int N, int K,
                    long long a_sm, long long a_sk, long long b_sk, long long b_sn, long long ldc,
                    int nb1, long long a_bs0, long long a_bs1, long long b_bs0, long long b_bs1,
                    long long c_bs0, long long c_bs1, const T* __restrict__ bias, const T* __restrict__ residual,
                    long long ldr, long long r_bs0, long long r_bs1, T* __restrict__ preact, int act, int bias_rows) {
  constexpr int TK = 16;
  __shared__ __align__(16) float As[TK][128 + 4];
  __shared__ __align__(16) float Bs[TK][128 + 4];
  const int b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
  A += b0 * a_bs0 + b1 * a_bs1;
  B += b0 * b_bs0 + b1 * b_bs1;
  const long long c_base = b0 * c_bs0 + b1 * c_bs1;
  const long long r_base = b0 * r_bs0 + b1 * r_bs1;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * 128;
  // Loader mapping: 2048 elements per operand tile, 8 per thread.  K-fast: 16 consecutive threads
  // walk the reduction; MN-fast: 128 consecutive threads walk the rows / columns.
  const bool a_kfast = a_sk == 1, b_kfast = b_sk == 1 && b_sn != 1;
  float ra[8], rb[8];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = tid + j * 256;
      const int ak = a_kfast ? (e & 15) : (e >> 7), am = a_kfast ? (e >> 4) : (e & 127);
      const int gm = m0 + am, gk = k0 + ak;
      ra[j] = (gm < M && gk < K) ? to_f(A[gm * a_sm + gk * a_sk]) : 0.f;
      const int bk = b_kfast ? (e & 15) : (e >> 7), bn = b_kfast ? (e >> 4) : (e & 127);
      const int gn = n0 + bn, gk2 = k0 + bk;
      rb[j] = (gn < N && gk2 < K) ? to_f(B[gk2 * b_sk + gn * b_sn]) : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = tid + j * 256;
      const int ak = a_kfast ? (e & 15) : (e >> 7), am = a_kfast ? (e >> 4) : (e & 127);
      As[ak][am] = ra[j];
      const int bk = b_kfast ? (e & 15) : (e >> 7), bn = b_kfast ? (e >> 4) : (e & 127);
      Bs[bk][bn] = rb[j];
    }
  };
  float acc[8][8] = {};
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += TK) {
    stash();
    __syncthreads();
    if (k0 + TK < K) fetch(k0 + TK);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float4 a_lo = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 a_hi = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
      const float4 b_lo = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float4 b_hi = *reinterpret_cast<const float4*>(&Bs[kk][64 + tx * 4]);
      const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      const float b[8] = {b_lo.x, b_lo.y, b_lo.z, b_lo.w, b_hi.x, b_hi.y, b_hi.z, b_hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= N) continue;
      float x = acc[i][j];
      if (bias) x += to_f(bias[bias_rows ? gm : gn]);
      if (preact) preact[c_base + gm * ldc + gn] = from_f<T>(act == 4 ? gelu_grad(x) : x);
      x = apply_act(x, act == 4 ? 2 : act);
      if (residual) {
        const float aux = to_f(residual[r_base + gm * ldr + gn]);
        x = (act == 3) ? x * aux : x + aux;
      }
      C[c_base + gm * ldc + gn] = from_f<T>(x);
    }
  }
}

// ------------------------------------------------------ float32 through tcgen05
// A float32 value x is the exact sum of three bfloat16 pieces: hi = bf16(x), mid = bf16(x - hi),
// lo = bf16(x - hi - mid).  A product a * b is then the sum of nine piece products, each exact in
// float32; the six largest (hi*hi, hi*mid, mid*hi, mid*mid, hi*lo, lo*hi) carry it to about
// 2^-23 relative.  Laying the pieces side by side along K turns the float32 GEMM into one
// bfloat16 GEMM with a six times longer reduction and float32 accumulation in tensor memory:
//   A' = [hi | hi | mid | mid | hi | lo]   (M x 6K)      B' = [hi | mid | hi | mid | lo | hi]   (N x 6K)
// This kernel writes one operand in that form, K-major and packed, from any strided source
// (tile transpose through shared memory keeps both sides coalesced).  ROLE 0 = A', 1 = B'.
template <int ROLE>
__global__ void split3_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int MN, int K, long long s_mn,
                              long long s_k, long long bs0, long long bs1, int nb1, int Kp, int mn_fast) {
  __shared__ float tile[32][33];  // [k][mn]
  const int b0 = blockIdx.z / nb1, b1 = blockIdx.z - b0 * nb1;
  src += b0 * bs0 + b1 * bs1;
  dst += static_cast<long long>(blockIdx.z) * MN * Kp;
  const int k0 = blockIdx.x * 32, mn0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int slow = ty + j * 8;
    const int k = k0 + (mn_fast ? slow : tx), mn = mn0 + (mn_fast ? tx : slow);
    const float x = (k < K && mn < MN) ? src[mn * s_mn + k * s_k] : 0.f;
    tile[mn_fast ? slow : tx][mn_fast ? tx : slow] = x;
  }
  __syncthreads();
  const int k = k0 + tx;
  if (k >= K) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int mn = mn0 + ty + j * 8;
    if (mn >= MN) continue;
    const float x = tile[tx][ty + j * 8];
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* row = dst + static_cast<long long>(mn) * Kp + k;
    if (ROLE == 0) {
      row[0] = hi; row[K] = hi; row[2LL * K] = mid; row[3LL * K] = mid; row[4LL * K] = hi; row[5LL * K] = lo;
    } else {
      row[0] = hi; row[K] = mid; row[2LL * K] = hi; row[3LL * K] = mid; row[4LL * K] = lo; row[5LL * K] = hi;
    }
  }
}

// Split-K second pass: C[m, n] = sum over s of partial[s, m, n] (float32 partials, fixed order).
template <class T>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, T* __restrict__ C, int splits, long long MN, int N, long long ldc) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < MN; i += stride * 4) {
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int sidx = 1; sidx < splits; ++sidx) {
      const float4 v = *reinterpret_cast<const float4*>(partial + sidx * MN + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long m = i / N;
    const int n = static_cast<int>(i - m * N);  // N is a multiple of 4: the four values share a row
    T* dst = C + m * ldc + n;
    dst[0] = from_f<T>(acc.x); dst[1] = from_f<T>(acc.y); dst[2] = from_f<T>(acc.z); dst[3] = from_f<T>(acc.w);
  }
}

// ---------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is unavailable in this driver");
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Encoded tensor maps are cached: a training step presents the same (pointer, extents, strides,
// box) combinations again and again (weights never move, activations come back from the pool at
// the same addresses), and each cuTensorMapEncodeTiled call costs the host about as much as
// the rest of a launch.  The cache is a flat hash table that is simply cleared when it fills up.
struct MapKey {
  const void* ptr;
  uint64_t dims[5];
  uint64_t strides[4];
  uint32_t box[5];
  uint32_t rank, dtype, promo;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) { h ^= w[i]; h *= 0xBF58476D1CE4E5B9ull; h ^= h >> 29; }
    return static_cast<size_t>(h);
  }
};
static_assert(sizeof(MapKey) % 8 == 0, "MapKey is hashed as 64-bit words");
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
std::atomic<long long> g_map_hits{0}, g_map_misses{0};

bool encode_cached(CUtensorMap* out, DType dt, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box, CUtensorMapL2promotion promo) {
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = base;
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  key.rank = static_cast<uint32_t>(rank);
  key.dtype = static_cast<uint32_t>(dt);
  key.promo = static_cast<uint32_t>(promo);
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      g_map_hits.fetch_add(1, std::memory_order_relaxed);
      return true;
    }
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = encode_fn()(out, dt == DType::BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                 static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  g_map_misses.fetch_add(1, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(g_map_mu);
  if (g_map_cache.size() >= 8192) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return true;
}

// Logical operand of the GEMM: `mn` x `k` elements with element strides, plus batch strides.
struct OperandView {
  const void* ptr;
  long long mn, k, s_mn, s_k, bs0, bs1;
  bool bcast;  // every batch entry reads the same matrix
};

bool tma_compatible(const OperandView& o, int nb0, int nb1) {
  if ((reinterpret_cast<uintptr_t>(o.ptr) & 15u) != 0) return false;
  const bool k_major = o.s_k == 1 || o.k == 1;
  const bool mn_major = o.s_mn == 1 || o.mn == 1;
  if (!k_major && !mn_major) return false;
  const long long other = (o.s_k == 1 || (o.k == 1 && o.s_mn != 1)) ? o.s_mn : o.s_k;
  if (other % 8 != 0 || other <= 0) return false;
  if (o.bcast) return true;
  if (nb1 > 1 && (o.bs1 % 8 != 0 || o.bs1 <= 0)) return false;
  if (nb0 > 1 && (o.bs0 % 8 != 0 || o.bs0 <= 0)) return false;
  return true;
}

// Builds a rank-4 tensor map {inner, rows, batch1, batch0}.  K-major: inner = K and the box
// is 64 x box_rows; MN-major: inner = MN and the box is 64 (MN) x 64 (K rows).
CUtensorMap make_map(const OperandView& o, bool mn_major, int box_rows, int nb0, int nb1, DType dt) {
  CUtensorMap m;
  const cuuint64_t inner = mn_major ? o.mn : o.k;
  const cuuint64_t rows = mn_major ? o.k : o.mn;
  const long long row_stride = mn_major ? o.s_k : o.s_mn;
  if (o.bcast) { nb0 = 1; nb1 = 1; }
  cuuint64_t dims[4] = {inner, rows, static_cast<cuuint64_t>(nb1), static_cast<cuuint64_t>(nb0)};
  // Strides of unit dims still have to be valid multiples of 16 bytes.
  const long long rs = rows > 1 ? row_stride : static_cast<long long>((inner + 7) / 8 * 8);
  const long long s1 = nb1 > 1 ? o.bs1 : rs * static_cast<long long>(rows);
  const long long s0 = nb0 > 1 ? o.bs0 : s1 * nb1;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(rs) * 2, static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s0) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(mn_major ? 64 : box_rows), 1, 1};
  if (!encode_cached(&m, dt, 4, o.ptr, dims, strides, box, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
    throw std::runtime_error("cuTensorMapEncodeTiled rejected a GEMM operand");
  return m;
}

std::mutex g_err_mu;
int* g_err_flag[64] = {};
int g_pair_clusters[64] = {};  // CTA pairs the device keeps resident at once (0 = not asked yet)

int* error_flag(int device) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  if (!g_err_flag[device]) {
    OB_CUDA(cudaMalloc(&g_err_flag[device], sizeof(int)));
    OB_CUDA(cudaMemset(g_err_flag[device], 0, sizeof(int)));
  }
  return g_err_flag[device];
}

struct Epilogue {
  Tensor bias, residual, preact;
  int act = 0;
  bool bias_rows = false;
};

template <class T>
void launch_simt(const OperandView& a, const OperandView& b, Tensor& C, int M, int N, int K, int nb0, int nb1,
                 long long ldc, long long c_bs0, long long c_bs1, const Epilogue& ep, cudaStream_t st, bool big) {
  const long long ldr = ep.residual.defined() ? ldc : 0;
  if (big) {  // the planner's choice: see plan_gemm
    dim3 grid128((N + 127) / 128, (M + 127) / 128, nb0 * nb1);
    gemm_simt128_kernel<T><<<grid128, 256, 0, st>>>(
        static_cast<const T*>(a.ptr), static_cast<const T*>(b.ptr), C.data_as<T>(), M, N, K, a.s_mn, a.s_k, b.s_k, b.s_mn, ldc,
        nb1, a.bs0, a.bs1, b.bs0, b.bs1, c_bs0, c_bs1, ep.bias.defined() ? ep.bias.data_as<T>() : nullptr,
        ep.residual.defined() ? ep.residual.data_as<T>() : nullptr, ldr, c_bs0, c_bs1,
        ep.preact.defined() ? ep.preact.data_as<T>() : nullptr, ep.act, ep.bias_rows ? 1 : 0);
    check_launch("gemm (SIMT 128x128)");
    return;
  }
  dim3 grid((N + 63) / 64, (M + 63) / 64, nb0 * nb1);
  gemm_simt_kernel<T><<<grid, dim3(16, 16), 0, st>>>(
      static_cast<const T*>(a.ptr), static_cast<const T*>(b.ptr), C.data_as<T>(), M, N, K, a.s_mn, a.s_k, b.s_k, b.s_mn, ldc,
      nb1, a.bs0, a.bs1, b.bs0, b.bs1, c_bs0, c_bs1, ep.bias.defined() ? ep.bias.data_as<T>() : nullptr,
      ep.residual.defined() ? ep.residual.data_as<T>() : nullptr, ldr, c_bs0, c_bs1,
      ep.preact.defined() ? ep.preact.data_as<T>() : nullptr, ep.act, ep.bias_rows ? 1 : 0);
  check_launch("gemm (SIMT)");
}

template <class T, int BN, int TM, int EW = kEpilogueWarps, bool PAIR = false>
void launch_tc05(const OperandView& a, const OperandView& b, bool a_mn, bool b_mn, Tensor& C, int M, int N, int K,
                 int nb0, int nb1, long long ldc, long long c_bs0, long long c_bs1, const Epilogue& ep, cudaStream_t st,
                 bool out_f32 = false, DType out_f32_operands = DType::BF16) {
  using L = SmemLayout<BN, TM, PAIR>;
  const DType dt = out_f32 ? out_f32_operands : C.dtype();  // operand type of the tensor maps
  const CUtensorMap ma = make_map(a, a_mn, TM, nb0, nb1, dt);
  const CUtensorMap mb = make_map(b, b_mn, PAIR ? BN / 2 : BN, nb0, nb1, dt);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.nb0 = nb0; p.nb1 = nb1; p.a_mn = a_mn; p.b_mn = b_mn;
  p.a_bc = a.bcast ? 1 : 0; p.b_bc = b.bcast ? 1 : 0; p.bias_rows = ep.bias_rows ? 1 : 0;
  p.C = C.data(); p.ldc = ldc; p.c_bs0 = c_bs0; p.c_bs1 = c_bs1;
  p.bias = ep.bias.defined() ? ep.bias.data() : nullptr;
  p.residual = ep.residual.defined() ? ep.residual.data() : nullptr;
  p.ldr = ldc; p.r_bs0 = c_bs0; p.r_bs1 = c_bs1;
  p.preact = ep.preact.defined() ? ep.preact.data() : nullptr;
  p.act = ep.act;
  p.err = error_flag(C.device().index);
  // Output tensor maps for the TMA-store epilogue (row-major [M, N] tiles of 64 x 32).
  auto out_map = [&](void* ptr, CUtensorMap* out) {
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 15u) || ldc % 8 != 0 || ldc < N || N % 8 != 0) return false;
    if (nb1 > 1 && (c_bs1 % 8 != 0 || c_bs1 <= 0)) return false;
    if (nb0 > 1 && (c_bs0 % 8 != 0 || c_bs0 <= 0)) return false;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(nb1), static_cast<cuuint64_t>(nb0)};
    const long long s1 = nb1 > 1 ? c_bs1 : ldc * static_cast<long long>(M);
    const long long s0 = nb0 > 1 ? c_bs0 : s1 * nb1;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(ldc) * 2, static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s0) * 2};
    cuuint32_t box[4] = {64, 32, 1, 1};
    return encode_cached(out, dt, 4, ptr, dims, strides, box, CU_TENSOR_MAP_L2_PROMOTION_NONE);
  };
  CUtensorMap mc = ma, mz = ma;
  static const bool direct_store = [] { const char* e = std::getenv("ORTHON_GEMM_STORE"); return e != nullptr && std::string(e) == "direct"; }();
  bool tma_store = !direct_store && !out_f32 && out_map(p.C, &mc);
  p.out_f32 = out_f32 ? 1 : 0;
  if (tma_store && p.preact != nullptr) tma_store = out_map(p.preact, &mz);
  if (tma_store && p.residual != nullptr &&
      ((reinterpret_cast<uintptr_t>(p.residual) & 15u) || p.ldr % 8 != 0 || p.r_bs0 % 8 != 0 || p.r_bs1 % 8 != 0)) tma_store = false;
  if (tma_store && p.bias != nullptr && (reinterpret_cast<uintptr_t>(p.bias) & 15u)) tma_store = false;
  p.tma_store = tma_store ? 1 : 0;
  static std::once_flag once;
  std::call_once(once, [] {
    OB_CUDA(cudaFuncSetAttribute(gemm_tc05_kernel<T, BN, TM, EW, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  });
  constexpr int kTileRows = PAIR ? 2 * TM : TM;
  const long long tiles = static_cast<long long>((M + kTileRows - 1) / kTileRows) * ((N + BN - 1) / BN) * nb0 * nb1;
  if (!PAIR) {
    const int grid = static_cast<int>(std::min<long long>(tiles, sm_count_for(C)));
    gemm_tc05_kernel<T, BN, TM, EW, PAIR><<<grid, gemm_threads(TM, EW), L::kTotal, st>>>(ma, mb, mc, mz, p);
    check_launch("gemm_tc05");
    return;
  }
  // Clusters of two CTAs; as many clusters as the device can keep resident at once (SMs that
  // cannot be paired inside their GPC stay idle), each walking the tile list with that stride.
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(gemm_threads(TM, EW));
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = st;
  int& resident = g_pair_clusters[C.device().index];
  if (resident == 0) {
    cfg.gridDim = dim3(2 * static_cast<unsigned>(sm_count_for(C) / 2));
    int n = 0;
    OB_CUDA(cudaOccupancyMaxActiveClusters(&n, gemm_tc05_kernel<T, BN, TM, EW, PAIR>, &cfg));
    resident = std::max(1, n);
  }
  cfg.gridDim = dim3(2 * static_cast<unsigned>(std::min<long long>(tiles, resident)));
  OB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc05_kernel<T, BN, TM, EW, PAIR>, ma, mb, mc, mz, p));
  check_launch("gemm_tc05 (CTA pairs)");
}


// Shared driver for Matmul and Linear.  `A`/`B` are the stored tensors, flags select op().
void gemm_dispatch(const Tensor& A_in, bool ta, const Tensor& B_in, bool tb, Tensor& C, const Epilogue& ep, cudaStream_t st) {
  Tensor A = A_in, B = B_in;
  const int nd = A.ndim();
  const int nbd = nd - 2;
  const int nb0 = nbd == 2 ? static_cast<int>(A.shape()[0]) : 1;
  const int nb1 = nbd >= 1 ? static_cast<int>(A.shape()[nbd - 1]) : 1;
  auto view_of = [&](const Tensor& t, bool trans, bool is_a) {
    OperandView o{};
    o.ptr = t.data();
    const long long rs = t.strides()[nbd], cs = t.strides()[nbd + 1];
    const long long r = t.shape()[nbd], c = t.shape()[nbd + 1];
    // op(t) logical: A' is [M, K]; B' is [K, N].
    const long long lr = trans ? c : r, lc = trans ? r : c, lrs = trans ? cs : rs, lcs = trans ? rs : cs;
    if (is_a) { o.mn = lr; o.k = lc; o.s_mn = lrs; o.s_k = lcs; }
    else { o.k = lr; o.mn = lc; o.s_k = lrs; o.s_mn = lcs; }
    o.bs0 = nbd == 2 ? t.strides()[0] : 0;
    o.bs1 = nbd >= 1 ? t.strides()[nbd - 1] : 0;
    o.bcast = nbd >= 1 && o.bs1 == 0 && (nbd < 2 || o.bs0 == 0) && (nb0 * nb1 > 1);
    return o;
  };
  OperandView a = view_of(A, ta, true), b = view_of(B, tb, false);
  const int M = static_cast<int>(a.mn), N = static_cast<int>(b.mn), K = static_cast<int>(a.k);
  const long long ldc = C.strides()[nbd];
  const long long c_bs0 = nbd == 2 ? C.strides()[0] : 0, c_bs1 = nbd >= 1 ? C.strides()[nbd - 1] : 0;
  const DType dt = C.dtype();

  GemmProblem prob;
  prob.dtype = dt;
  prob.m = M; prob.n = N; prob.k = K;
  prob.batch = static_cast<int64_t>(nb0) * nb1;
  prob.has_bias = ep.bias.defined(); prob.has_residual = ep.residual.defined(); prob.has_preact = ep.preact.defined();
  prob.act = ep.act;
  prob.tcgen05 = Runtime::instance().cuda(C.device().index).supports_tcgen05();
  prob.sms = sm_count_for(C);
  GemmPlanOptions opts = plan_options();
  if (dt != DType::F32 && prob.tcgen05 && opts.force_route != 1 && (static_cast<long long>(M) * N * K >= (1LL << 18) || opts.force_route == 2)) {
    // Operands that TMA cannot describe are packed once (the packed copy is K-major).
    if (!tma_compatible(a, nb0, nb1)) {
      A = Tensor::empty(A.shape(), A.dtype(), A.device());
      strided_copy_cuda(A_in, A, st);
      a = view_of(A, ta, true);
    }
    if (!tma_compatible(b, nb0, nb1)) {
      B = Tensor::empty(B.shape(), B.dtype(), B.device());
      strided_copy_cuda(B_in, B, st);
      b = view_of(B, tb, false);
    }
    prob.tma_ok = tma_compatible(a, nb0, nb1) && tma_compatible(b, nb0, nb1);
  }
  GemmPlan plan = plan_gemm(prob, opts);
  const bool a_mn = !(a.s_k == 1 || (a.k == 1 && a.s_mn != 1));
  const bool b_mn = !(b.s_k == 1 || (b.k == 1 && b.s_mn != 1));
  if (plan.route == GemmRoute::Tc05SplitK) {
    // The K slices run as batch entries of the same kernel (the slice index is a batch stride along
    // K); float32 partials go to scratch and a second pass adds them in a fixed order.
    const int splits = plan.splits;
    const long long Ks = K / splits;
    OperandView as = a, bs = b;
    as.k = Ks; bs.k = Ks;
    as.bs1 = Ks * a.s_k; bs.bs1 = Ks * b.s_k;
    as.bs0 = 0; bs.bs0 = 0;
    as.bcast = false; bs.bcast = false;
    if (tma_compatible(as, 1, splits) && tma_compatible(bs, 1, splits)) {
      Tensor partial = Tensor::empty({static_cast<int64_t>(splits), static_cast<int64_t>(M), static_cast<int64_t>(N)}, DType::F32, C.device());
      Epilogue none;
      const long long mn = static_cast<long long>(M) * N;
      g_last_route.store(static_cast<int>(plan.route), std::memory_order_relaxed);
      g_last_plan_bn.store(plan.bn, std::memory_order_relaxed);
#define OB_SPLITK_LAUNCH(TT)                                                                                                   \
  do {                                                                                                                         \
    if (plan.bn == 256) launch_tc05<TT, 256, 128>(as, bs, a_mn, b_mn, partial, M, N, static_cast<int>(Ks), 1, splits, N, 0, mn, none, st, true, dt); \
    else launch_tc05<TT, 128, 128>(as, bs, a_mn, b_mn, partial, M, N, static_cast<int>(Ks), 1, splits, N, 0, mn, none, st, true, dt);      \
    splitk_reduce_kernel<TT><<<ew_grid(mn / 4 + 1, 256, prob.sms), 256, 0, st>>>(                                             \
        partial.data_as<float>(), C.data_as<TT>(), splits, mn, N, ldc);                                                        \
  } while (0)
      if (dt == DType::BF16) OB_SPLITK_LAUNCH(__nv_bfloat16);
      else OB_SPLITK_LAUNCH(__half);
#undef OB_SPLITK_LAUNCH
      check_launch("gemm_tc05 (split-K)");
      return;
    }
    opts.splitk = false;  // the slices are not TMA-describable: plan again without them
    plan = plan_gemm(prob, opts);
  }
  g_last_route.store(static_cast<int>(plan.route), std::memory_order_relaxed);
  g_last_plan_bn.store(plan.bn, std::memory_order_relaxed);
  switch (plan.route) {
    case GemmRoute::Simt64:
    case GemmRoute::Simt128:
      if (dt == DType::F32) launch_simt<float>(a, b, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st, plan.route == GemmRoute::Simt128);
      else if (dt == DType::BF16) launch_simt<__nv_bfloat16>(a, b, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st, plan.route == GemmRoute::Simt128);
      else launch_simt<__half>(a, b, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st, plan.route == GemmRoute::Simt128);
      return;
    case GemmRoute::Tc05Float32: {
      // A' = [hi | hi | mid | mid | hi | lo], B' = [hi | mid | hi | mid | lo | hi] along K (see split3_kernel).
      const int Kp = static_cast<int>((static_cast<long long>(K) * 6 + 7) / 8 * 8);
      auto split_operand = [&](const OperandView& o, int role, Tensor& holder) {
        const int nb = o.bcast ? 1 : nb0 * nb1;
        holder = Tensor::empty({static_cast<int64_t>(nb), o.mn, static_cast<int64_t>(Kp)}, DType::BF16, C.device());
        if (Kp != K * 6) OB_CUDA(cudaMemsetAsync(holder.data(), 0, holder.nbytes(), st));
        const int mn_fast = (o.s_mn == 1 && o.s_k != 1) ? 1 : 0;
        dim3 grid(static_cast<unsigned>((o.k + 31) / 32), static_cast<unsigned>((o.mn + 31) / 32), static_cast<unsigned>(nb));
        auto* dst = static_cast<__nv_bfloat16*>(holder.data());
        const auto* src = static_cast<const float*>(o.ptr);
        const long long sb0 = o.bcast ? 0 : o.bs0, sb1 = o.bcast ? 0 : o.bs1;
        const int inner_nb = o.bcast ? 1 : nb1;
        if (role == 0) split3_kernel<0><<<grid, dim3(32, 8), 0, st>>>(src, dst, static_cast<int>(o.mn), static_cast<int>(o.k), o.s_mn, o.s_k, sb0, sb1, inner_nb, Kp, mn_fast);
        else split3_kernel<1><<<grid, dim3(32, 8), 0, st>>>(src, dst, static_cast<int>(o.mn), static_cast<int>(o.k), o.s_mn, o.s_k, sb0, sb1, inner_nb, Kp, mn_fast);
        check_launch("gemm float32 split");
        OperandView v{};
        v.ptr = holder.data();
        v.mn = o.mn; v.k = Kp; v.s_mn = Kp; v.s_k = 1;
        v.bs1 = o.bcast ? 0 : o.mn * static_cast<long long>(Kp);
        v.bs0 = o.bcast ? 0 : v.bs1 * nb1;
        v.bcast = o.bcast;
        return v;
      };
      Tensor a_pieces, b_pieces;
      if (a.mn > 65535LL * 32 || b.mn > 65535LL * 32) throw std::invalid_argument("matmul: float32 operand too tall for the split kernel grid");
      const OperandView a6 = split_operand(a, 0, a_pieces), b6 = split_operand(b, 1, b_pieces);
      if (plan.bn == 256) launch_tc05<__nv_bfloat16, 256, 128>(a6, b6, false, false, C, M, N, Kp, nb0, nb1, ldc, c_bs0, c_bs1, ep, st, true);
      else launch_tc05<__nv_bfloat16, 128, 128>(a6, b6, false, false, C, M, N, Kp, nb0, nb1, ldc, c_bs0, c_bs1, ep, st, true);
      return;
    }
    default:
      break;
  }
  const bool pair = plan.route == GemmRoute::Tc05Pair;
#define OB_GEMM_LAUNCH(TT)                                                                                                    \
  do {                                                                                                                        \
    if (pair && plan.tm == 256) launch_tc05<TT, 256, 256, 4, true>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st); \
    else if (pair && plan.epilogue_warps == 8) launch_tc05<TT, 256, 128, 8, true>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st); \
    else if (pair) launch_tc05<TT, 256, 128, 4, true>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st);      \
    else if (plan.tm == 256) launch_tc05<TT, 256, 256>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st);     \
    else if (plan.bn == 256 && plan.epilogue_warps == 8) launch_tc05<TT, 256, 128, 8>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st); \
    else if (plan.bn == 256) launch_tc05<TT, 256, 128>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st);     \
    else launch_tc05<TT, 128, 128>(a, b, a_mn, b_mn, C, M, N, K, nb0, nb1, ldc, c_bs0, c_bs1, ep, st);                         \
  } while (0)
  if (dt == DType::BF16) OB_GEMM_LAUNCH(__nv_bfloat16);
  else OB_GEMM_LAUNCH(__half);
#undef OB_GEMM_LAUNCH
}

void k_matmul(OpCall& c) {
  Epilogue ep;
  gemm_dispatch(c.in[0], c.i[0] != 0, c.in[1], c.i[1] != 0, c.out[0], ep, stream_of(c));
}

void k_linear(OpCall& c) {
  Epilogue ep;
  ep.bias = c.in[2];
  ep.residual = c.in[3];
  ep.preact = c.out[1];
  ep.act = static_cast<int>(c.i[0]);
  gemm_dispatch(c.in[0], false, c.in[1], false, c.out[0], ep, stream_of(c));
}

}  // namespace

// GEMM entry for other kernels of the backend (convolution lowers to it).
void gemm_launch(const Tensor& A, bool ta, const Tensor& B, bool tb, Tensor& C, const Tensor& bias, bool bias_rows,
                 cudaStream_t st) {
  Epilogue ep;
  ep.bias = bias;
  ep.bias_rows = bias_rows;
  gemm_dispatch(A, ta, B, tb, C, ep, st);
}

// Shared with the other tcgen05 kernels of the backend: the per-device error word that bounded
// waits report into, and a rank-N 128-byte-swizzled tiled tensor map over 16-bit elements
// (dims/box innermost first, strides in bytes for dims 1..rank-1).
int* tc05_error_flag(int device) { return error_flag(device); }

bool tc05_encode_map(CUtensorMap* out, DType dt, int rank, void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box) {
  cuuint64_t d[5], s[4];
  cuuint32_t b[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  return encode_cached(out, dt, rank, base, d, s, b, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

// CTA pairs of the pair-form GEMM that are resident at once on `device` (0 before its first launch).
int gemm_pair_clusters(int device) { return g_pair_clusters[device]; }

// (hits, misses) of the tensor-map cache since the process started.
void tensor_map_cache_stats(long long* hits, long long* misses) {
  *hits = g_map_hits.load(std::memory_order_relaxed);
  *misses = g_map_misses.load(std::memory_order_relaxed);
}

// Diagnostics (reference project: src/diagnostics/matmul.cpp:14-87): force a route, read the
// route the last matmul took.
void set_gemm_route(int route) { g_force_route.store(route, std::memory_order_relaxed); }
void set_float32_matmul_precision(int level) { g_f32_precision.store(level ? 1 : 0, std::memory_order_relaxed); }
int float32_matmul_precision() { return f32_precision(); }
void set_gemm_pair_mode(int mode) { g_pair_mode.store(mode, std::memory_order_relaxed); }
// Route of the last product in the numbering the diagnostics expose: 1 = SIMT, 2 = tcgen05 with
// 128-column tiles, 3 = tcgen05 with 256-column tiles, 4 = tcgen05 CTA pairs.
int last_gemm_route() {
  const int route = g_last_route.load(std::memory_order_relaxed);
  if (route == 0) return 0;
  if (route <= static_cast<int>(GemmRoute::Simt128)) return 1;
  if (route == static_cast<int>(GemmRoute::Tc05Pair)) return 4;
  return g_last_plan_bn.load(std::memory_order_relaxed) == 256 ? 3 : 2;
}

// Reads and clears the GEMM error word of a device (0 = no error).  Synchronizes the device.
int take_gemm_error(int device) {
  int* flag;
  {
    std::lock_guard<std::mutex> lock(g_err_mu);
    flag = g_err_flag[device];
  }
  if (!flag) return 0;
  int host = 0;
  OB_CUDA(cudaMemcpy(&host, flag, sizeof(int), cudaMemcpyDeviceToHost));
  if (host) OB_CUDA(cudaMemset(flag, 0, sizeof(int)));
  return host;
}

void register_cuda_gemm(KernelRegistry& r) {
  const uint8_t any = kContiguous | kStrided | kEmpty;
  r.add_kernel(OperatorId::Matmul, Constraints{Backend::CUDA, kMaskF32, any, Capability::None}, k_matmul, "sm100_gemm_simt_f32");
  r.add_kernel(OperatorId::Matmul, Constraints{Backend::CUDA, dtype_bit(DType::F16), any, Capability::None}, k_matmul, "sm100_gemm_tc05_f16");
  r.add_kernel(OperatorId::Matmul, Constraints{Backend::CUDA, dtype_bit(DType::BF16), any, Capability::Bf16}, k_matmul, "sm100_gemm_tc05_bf16");
  r.add_kernel(OperatorId::Linear, Constraints{Backend::CUDA, kMaskF32, any, Capability::None}, k_linear, "sm100_linear_simt_f32");
  r.add_kernel(OperatorId::Linear, Constraints{Backend::CUDA, dtype_bit(DType::F16), any, Capability::None}, k_linear, "sm100_linear_tc05_f16");
  r.add_kernel(OperatorId::Linear, Constraints{Backend::CUDA, dtype_bit(DType::BF16), any, Capability::Bf16}, k_linear, "sm100_linear_tc05_bf16");
}

}  // namespace cu
}  // namespace ob

// attention_tc05: fused multi-head self-attention on the 5th-generation tensor cores (sm_100a).
//
// Input is the packed projection qkv[B, T, 3E] (E = H*D, head h of q/k/v at columns
// {0,E,2E} + h*D); heads are read in place through one rank-3 tensor map, nothing is split,
// transposed or packed, and the [T, T] score matrix never exists in global memory.
//
//   forward : O = softmax(scale * Q K^T + causal mask) V, LSE[b,h,t] = log sum exp (natural log)
//   backward: dQ, dK, dV from (qkv, O, LSE, dO) with the probabilities recomputed tile by tile
//
// Forward design (one CTA = one (batch, head) and 256 query rows, 320 threads):
//   warp 0      TMA producer: Q (two 128-row tiles, once), then K_j / V_j tiles of 64 keys through
//               two 4-stage rings
//   warp 1      one thread issues tcgen05.mma: S_w = Q_w K_j^T (TMEM, 64 fp32 columns per query
//               tile) and O_w += P_w V_j (TMEM, D columns per query tile)
//   warps 2-5   softmax group 0, warps 6-9 softmax group 1: one thread per query row reads its
//               S row from TMEM, keeps the running max / sum (online softmax, base-2 exponent),
//               rescales the O accumulator in TMEM when the max moved, writes P as bf16/f16 into
//               128-byte-swizzled shared memory (the A operand of the second MMA)
//   The two groups work on alternating MMAs (S_1 and P_0 V run while group 0 is in softmax and
//   vice versa), so the tensor pipe and the exponent unit overlap.
// Backward is two kernels so that every output element has exactly one writer (deterministic,
// no atomics): one CTA per key tile accumulates dK and dV over query tiles; one CTA per query
// tile accumulates dQ over key tiles.  Both recompute S and dP = dO V^T on the tensor cores.
//
// Every mbarrier wait is bounded (clock budget -> error word, unwind, TMEM released).
//
// Replaces (reference project paths): python/orthon/functional/math.py:39-72 (composed
// matmul / log_softmax / exp / matmul attention) and python/orthon/nn/attention.py:84-103
// (head split by reshape + transpose + contiguous).
#include <cuda.h>

#include <cstdio>

#include <mutex>

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

enum : int { kErrAttnProducer = 11, kErrAttnMma = 12, kErrAttnSoftmax = 13 };

constexpr int kTile = 128;  // query rows per softmax group and keys per K/V tile

struct FlashParams {
  int B, H, T, E;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  float scale;       // softmax scale
  float* lse;        // [B, H, T]
  const float* delta;  // [B, H, T] (backward): sum_d dO * O
  int* err;
  // Optional timeline of CTA (0, 0) of the dK/dV kernel: trace[it * 8 + slot] = clock64() at a phase
  // boundary (ORTHON_ATTENTION_TRACE=1 prints it after the launch).  Null in normal runs.
  long long* trace;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Bounded wait whose verdict is uniform across the warp (lanes may otherwise disagree right at
// the timeout, and the softmax warps use warp-collective instructions afterwards).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, err, code));
}

// Packs 8 floats into 8 16-bit values (one 16-byte chunk).
template <class T>
__device__ __forceinline__ uint4 pack8(const float* v) {
  Pack<T> p;
#pragma unroll
  for (int j = 0; j < 8; ++j) p.v[j] = from_f<T>(v[j]);
  return *reinterpret_cast<uint4*>(&p);
}

// ------------------------------------------------------------------ forward
constexpr int kKeys = 64;  // keys per K / V tile of the forward kernel

// Q (two 128-row tiles) stays resident; K and V stream through rings of kStages 64-key tiles each
// (deep enough that the TMA latency of about 5000 cycles hides behind the MMAs of the tiles in
// between); P holds one [128 x 64] probability tile per softmax group.
template <int D>
struct FwdSmem {
  static constexpr int kQBytes = kTile * D * 2;        // one query tile
  static constexpr int kKVBytes = kKeys * D * 2;       // one K or V tile
  static constexpr int kPBytes = kTile * kKeys * 2;    // one probability tile
  static constexpr int kStages = 4;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kQBytes;
  static constexpr int kVOff = kKOff + kStages * kKVBytes;
  static constexpr int kPOff = kVOff + kStages * kKVBytes;
  static constexpr int kBarOff = kPOff + 2 * kPBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;  // +1024 for manual alignment
  static_assert(kTotal <= 232448, "exceeds the shared memory of one CTA");
};

constexpr int kFwdThreads = 320;

template <class T, int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q128, const __grid_constant__ CUtensorMap map_kv64,
                 const __grid_constant__ CUtensorMap map_o, FlashParams p) {
  using L = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                      // 1
  uint64_t* k_full = q_full + 1;                // kStages
  uint64_t* k_empty = k_full + L::kStages;
  uint64_t* v_full = k_empty + L::kStages;      // kStages
  uint64_t* v_empty = v_full + L::kStages;
  uint64_t* s_full = v_empty + L::kStages;      // 2
  uint64_t* p_full = s_full + 2;                // 2
  uint64_t* o_done = p_full + 2;                // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh - b * p.H;
  const int n_pairs = gridDim.y;
  const int pair = n_pairs - 1 - static_cast<int>(blockIdx.y);  // heaviest (latest rows) first for every head
  const int n_qtiles = (p.T + kTile - 1) / kTile;
  const int n_ktiles = (p.T + kKeys - 1) / kKeys;
  // Number of key tiles each query tile needs (the causal mask ends at the tile's last row).
  auto tiles_for = [&](int w) {
    const int qt = 2 * pair + w;
    return (qt >= n_qtiles) ? 0 : (p.causal ? min(n_ktiles, 2 * qt + 2) : n_ktiles);
  };
  const int n_w0 = tiles_for(0), n_w1 = tiles_for(1);
  const int n_kv = max(n_w0, n_w1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) { mbar_init(&s_full[w], 1); mbar_init(&p_full[w], 4); mbar_init(&o_done[w], 1); }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_s = [&](int w) { return tmem_base + static_cast<uint32_t>(w) * kKeys; };
  auto tmem_o = [&](int w) { return tmem_base + 2u * kKeys + static_cast<uint32_t>(w) * D; };

  const int col_q = h * D, col_k = p.E + h * D, col_v = 2 * p.E + h * D;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0 && n_kv > 0) {
      mbar_expect_tx(q_full, 2 * L::kQBytes);
#pragma unroll
      for (int w = 0; w < 2; ++w)
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(smem + L::kQOff + w * L::kQBytes + c * (kTile * 128), &map_q128, q_full, col_q + c * 64,
                      (2 * pair + w) * kTile, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % L::kStages;
        const uint32_t parity = ((j / L::kStages) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], parity, p.err, kErrAttnProducer)) break;
        mbar_expect_tx(&k_full[st], L::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(smem + L::kKOff + st * L::kKVBytes + c * (kKeys * 128), &map_kv64, &k_full[st], col_k + c * 64, j * kKeys, b);
        if (!mbar_wait(&v_empty[st], parity, p.err, kErrAttnProducer)) break;
        mbar_expect_tx(&v_full[st], L::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(smem + L::kVOff + st * L::kKVBytes + c * (kKeys * 128), &map_kv64, &v_full[st], col_v + c * 64, j * kKeys, b);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_kv > 0) {
      const bool bf = std::is_same<T, __nv_bfloat16>::value;
      const uint32_t idesc_s = make_idesc(bf, 0, 0, kTile, kKeys);  // S = Q K^T  (both K-major)
      const uint32_t idesc_o = make_idesc(bf, 0, 1, kTile, D);      // O = P V    (V is MN-major)
      // Base descriptors once; every MMA then costs two adds (see desc_advance).
      const uint64_t dq_base = make_desc(smem_u32(smem + L::kQOff), 16, 1024);
      const uint64_t dk_base = make_desc(smem_u32(smem + L::kKOff), 16, 1024);
      const uint64_t dp_base = make_desc(smem_u32(smem + L::kPOff), 16, 1024);
      const uint64_t dv_base = make_desc(smem_u32(smem + L::kVOff), kKeys * 128, 1024);
      auto issue_s = [&](int w, int st) {
        const uint64_t dq = desc_advance(dq_base, w * L::kQBytes), dk = desc_advance(dk_base, st * L::kKVBytes);
        const uint32_t d = tmem_s(w);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr int kBlockA = kTile * 128, kBlockB = kKeys * 128;
          umma_f16(d, desc_advance(dq, (kk / 4) * kBlockA + (kk % 4) * 32), desc_advance(dk, (kk / 4) * kBlockB + (kk % 4) * 32),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[w]);
      };
      auto issue_o = [&](int w, int st, bool accumulate) {
        const uint64_t dp = desc_advance(dp_base, w * L::kPBytes), dv = desc_advance(dv_base, st * L::kKVBytes);
        const uint32_t d = tmem_o(w);
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk)
          umma_f16(d, desc_advance(dp, kk * 32), desc_advance(dv, kk * 2048), idesc_o, (accumulate || kk > 0) ? 1u : 0u);
        umma_commit(&o_done[w]);
      };
      bool ok = mbar_wait(q_full, 0, p.err, kErrAttnMma);
      if (ok) ok = mbar_wait(&k_full[0], 0, p.err, kErrAttnMma);
      if (ok) {
        tc_fence_after();
        if (n_w0 > 0) issue_s(0, 0);
        if (n_w1 > 0) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % L::kStages, st_next = (j + 1) % L::kStages;
        if (!mbar_wait(&v_full[st], (j / L::kStages) & 1, p.err, kErrAttnMma)) { ok = false; break; }
        bool k_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          const int n_w = w ? n_w1 : n_w0;
          if (j < n_w) {
            if (!mbar_wait(&p_full[w], j & 1, p.err, kErrAttnMma)) { ok = false; break; }
            tc_fence_after();
            issue_o(w, st, j > 0);
          }
          if (j + 1 < n_w) {
            if (!k_ready) {
              if (!mbar_wait(&k_full[st_next], ((j + 1) / L::kStages) & 1, p.err, kErrAttnMma)) { ok = false; break; }
              tc_fence_after();
              k_ready = true;
            }
            issue_s(w, st_next);  // P_w ready implies S_w has been read out
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[st]);
        if (j + 1 < n_kv) umma_commit(&k_empty[st_next]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax groups
    const int w = (warp - 2) >> 2;        // query tile within the pair
    const int quarter = warp & 3;         // TMEM lane quarter of this warp
    const int r = quarter * 32 + lane;    // row within the query tile
    const int q_tile0 = (2 * pair + w) * kTile;
    const int q_row = q_tile0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* sp = smem + L::kPOff + w * L::kPBytes;
    const int n_it = w ? n_w1 : n_w0;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_it && ok; ++j) {
      if (!warp_wait(&s_full[w], j & 1, p.err, kErrAttnSoftmax)) { ok = false; break; }
      tc_fence_after();
      float s[kKeys];
      tmem_ld32_nowait(tmem_s(w) + lane_off, s);
      tmem_ld32_nowait(tmem_s(w) + lane_off + 32, s + 32);
      tmem_ld_wait();
      // Mask: keys past the sequence end, and keys after the query on tiles that reach the diagonal.
      const int key0 = j * kKeys;
      const bool diag = p.causal && (key0 + kKeys - 1 > q_tile0);
      if (diag || key0 + kKeys > p.T) {
        const int limit = diag ? min(q_row, p.T - 1) : p.T - 1;  // last visible key
#pragma unroll
        for (int c = 0; c < kKeys; ++c)
          if (key0 + c > limit) s[c] = -INFINITY;
      }
      float mx4[4] = {s[0], s[1], s[2], s[3]};  // four independent chains instead of one of 64
#pragma unroll
      for (int c = 4; c < kKeys; c += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(mx4[i], s[c + i]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // `m` is the exponent offset in use (log2 units), not necessarily the running maximum: it is
      // only moved, together with a rescale of the O accumulator, when some row of the warp has
      // grown past it by more than 2^8.  Until then p = 2^(s - m) stays below 256, which both
      // 16-bit formats hold, and the row sum and O stay consistent, so the result is unchanged;
      // the TMEM round trip of the rescale leaves the per-tile critical path.
      float m_cand = fmaxf(m, mx * p.scale_log2);
      if (m_cand == -INFINITY) m_cand = 0.f;  // fully masked row (rows past the sequence end)
      const bool move = (j == 0) || __any_sync(0xffffffffu, m_cand > m + 8.f);
      const float m_new = move ? m_cand : m;
      const float alpha = move ? fast_exp2(m - m_new) : 1.f;
      if (j > 0) {
        // P_{j-1} V has finished: the O accumulator is consistent and the P tile is free.
        if (!warp_wait(&o_done[w], (j - 1) & 1, p.err, kErrAttnSoftmax)) { ok = false; break; }
        tc_fence_after();
        if (move) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            float o[32];
            tmem_ld32(tmem_o(w) + lane_off + c * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(tmem_o(w) + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c8 = 0; c8 < kKeys / 8; ++c8) {
        float pv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pv[i] = fast_exp2(fmaf(s[c8 * 8 + i], p.scale_log2, -m_new));
          sum4[i & 3] += pv[i];
        }
        *reinterpret_cast<uint4*>(sp + sw128_offset(r, c8)) = pack8<T>(pv);
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m = m_new;
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[w]);
    }
    if (ok && n_it > 0 && warp_wait(&o_done[w], (n_it - 1) & 1, p.err, kErrAttnSoftmax)) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      // Every MMA of this query tile has finished, so its Q tile is idle: stage this warp's 32 rows
      // there and store them with TMA.
      uint8_t* so = smem + L::kQOff + w * L::kQBytes;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld32(tmem_o(w) + lane_off + c * 32, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= inv_l;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(so + (c / 2) * (kTile * 128) + sw128_offset(r, (c % 2) * 4 + q)) = pack8<T>(o + q * 8);
      }
      fence_async_smem();
      __syncwarp();
      const int store_row = q_tile0 + quarter * 32;
      if (lane == 0 && store_row < p.T) {  // rows past the end of a partly covered box are clipped by TMA
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_store_3d(&map_o, so + c * (kTile * 128) + quarter * 32 * 128, h * D + c * 64, store_row, b);
        tma_store_wait_all();
      }
      if (q_row < p.T) p.lse[(static_cast<long long>(b) * p.H + h) * p.T + q_row] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ----------------------------------------------------------------- backward
// delta[b, h, t] = sum_d dO[b, t, h*D + d] * O[b, t, h*D + d]; D/8 lanes per (b, t, h) row, 16-byte loads.
template <class T>
__global__ void attn_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out, float* __restrict__ delta, int B, int Tn,
                                  int H, int D) {
  const int lanes = D / 8;  // 8 or 16
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = tid / lanes;  // (b*T + t)*H + h, which is also the row of the [B*T*H, D] view
  const int sub = static_cast<int>(tid - row * lanes);
  const long long total = static_cast<long long>(B) * Tn * H;
  float acc = 0.f;
  if (row < total) {
    const Pack<T> a = load_pack(dout + row * D + sub * 8), o = load_pack(out + row * D + sub * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += to_f(a.v[k]) * to_f(o.v[k]);
  }
  for (int off = lanes / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < total && sub == 0) {
    const int h = static_cast<int>(row % H);
    const long long bt = row / H;
    const long long b = bt / Tn, t = bt - b * Tn;
    delta[(b * H + h) * Tn + t] = acc;
  }
}

// The conversion of scores into P / dS is latency-bound (TMEM loads, shuffles, shared-memory
// stores and barrier hand-offs per tile), so the 64 columns of a step are spread over four
// groups of four warps: each warp has half the serial work of a two-group split and twice as
// many warps hide each other's stalls.
constexpr int kBwdGroups = 4;
constexpr int kCG = 64 / kBwdGroups;  // columns of the streamed sub-tile per group
constexpr int kBwdThreads = 32 * (2 + 4 * kBwdGroups);  // TMA warp, MMA warp, the softmax groups
constexpr int kSub = 64;  // rows of the streamed operand per step (N of the score MMAs)

// Shared-memory plan of the backward kernels: two resident [128 x D] tiles, a ring of streamed
// [64 x D] tile pairs (deep enough to hide the TMA latency behind the MMAs of the other ring
// slots), and OPS double-buffered [128 x 64] operand tiles written by the softmax warps.
template <int D, int OPS, int NBUF, int STAGES>
struct BwdSmem {
  static constexpr int kBigBytes = kTile * D * 2;   // resident tile
  static constexpr int kSubBytes = kSub * D * 2;    // streamed tile
  static constexpr int kOpBytes = kTile * kSub * 2; // operand tile written by the softmax warps
  static constexpr int kStages = STAGES;
  static constexpr int kBigOff = 0;                                   // two resident tiles
  static constexpr int kRingOff = kBigOff + 2 * kBigBytes;            // kStages x (two streamed tiles)
  static constexpr int kOpBufs = NBUF;
  static constexpr int kOpOff = kRingOff + kStages * 2 * kSubBytes;   // [NBUF buffers][OPS tiles]
  static constexpr int kBarOff = kOpOff + NBUF * OPS * kOpBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
  static_assert(kTotal <= 232448, "exceeds the shared memory of one CTA");
};
// P^T / dS^T never touch shared memory: each softmax group packs its 16 columns to 16-bit pairs and
// writes them over its own score columns in tensor memory, from where the accumulate MMAs read
// them as the A operand.  That halves the shared-memory bytes per step (the limit of these
// short-N products) and leaves room for a five-deep ring.
template <int D> using DkvSmem = BwdSmem<D, 0, 0, 5>;
template <int D> using DqSmem = BwdSmem<D, 0, 0, 5>;

// dK, dV: one CTA per (batch, head, 128-key tile); streams 64-row query tiles.
//   S^T = K Q^T, dP^T = V dO^T (TMEM, 64 columns each, double buffered); one thread per key row
//   turns them into P^T and dS^T, packed to 16 bits over its own score columns (TMEM), which the
//   accumulate MMAs read as their A operand; dV += P^T dO, dK += dS^T Q (TMEM).
template <class T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_qkv128, const __grid_constant__ CUtensorMap map_qkv64,
                     const __grid_constant__ CUtensorMap map_do64, const __grid_constant__ CUtensorMap map_dqkv, FlashParams p) {
  using L = DkvSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* ring_full = kv_full + 1;
  uint64_t* ring_empty = ring_full + L::kStages;
  uint64_t* sdp_full = ring_empty + L::kStages;  // 2
  uint64_t* pds_full = sdp_full + 2;             // 2
  uint64_t* pds_free = pds_full + 2;             // 2
  uint64_t* acc_done = pds_free + 2;
  uint64_t* acc_step = acc_done + 1;             // 2, trace only: accumulate MMAs of a step complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_step + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long* const trace = (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) ? p.trace : nullptr;
  auto stamp = [&](int it, int slot) { if (trace != nullptr && it < 32) trace[it * 8 + slot] = clock64(); };
  const int bh = blockIdx.x, b = bh / p.H, h = bh - b * p.H;
  const int jt = blockIdx.y;                 // key tile (128 keys); tile 0 is the heaviest under the causal mask
  const int key0 = jt * kTile;
  const int n_sub = (p.T + kSub - 1) / kSub;  // query sub-tiles in the sequence
  const int i0 = p.causal ? (key0 / kSub) : 0;
  const int n_it = max(0, n_sub - i0);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&ring_full[s], 1); mbar_init(&ring_empty[s], 1); }
    for (int w = 0; w < 2; ++w) { mbar_init(&sdp_full[w], 1); mbar_init(&pds_full[w], 4 * kBwdGroups); mbar_init(&pds_free[w], 1); }
    mbar_init(acc_done, 1);
    mbar_init(&acc_step[0], 1); mbar_init(&acc_step[1], 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 256 + D;
  const int col_q = h * D, col_k = p.E + h * D, col_v = 2 * p.E + h * D;
  uint8_t* sk = smem + L::kBigOff;
  uint8_t* sv = sk + L::kBigBytes;

  if (warp == 0) {
    if (lane == 1 && trace != nullptr) {  // observer: completion time of each step's accumulate MMAs
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait(&acc_step[it & 1], (it >> 1) & 1, p.err, kErrAttnProducer)) break;
        stamp(it, 6);
      }
    }
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * L::kBigBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_3d(sk + c * (kTile * 128), &map_qkv128, kv_full, col_k + c * 64, key0, b);
        tma_load_3d(sv + c * (kTile * 128), &map_qkv128, kv_full, col_v + c * 64, key0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % L::kStages;
        if (!mbar_wait(&ring_empty[st], ((it / L::kStages) & 1) ^ 1, p.err, kErrAttnProducer)) break;
        stamp(it, 0);  // producer: ring slot free, loads issued
        mbar_expect_tx(&ring_full[st], 2 * L::kSubBytes);
        uint8_t* sq = smem + L::kRingOff + st * 2 * L::kSubBytes;
        uint8_t* sdo = sq + L::kSubBytes;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_3d(sq + c * (kSub * 128), &map_qkv64, &ring_full[st], col_q + c * 64, (i0 + it) * kSub, b);
          tma_load_3d(sdo + c * (kSub * 128), &map_do64, &ring_full[st], col_q + c * 64, (i0 + it) * kSub, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      const bool bf = std::is_same<T, __nv_bfloat16>::value;
      const uint32_t idesc_s = make_idesc(bf, 0, 0, kTile, kSub);  // [128 keys x 64 queries], both K-major
      const uint32_t idesc_a = make_idesc(bf, 0, 1, kTile, D);     // [128 keys x D], B operand MN-major
      const uint64_t dk_base = make_desc(smem_u32(sk), 16, 1024), dv_base = make_desc(smem_u32(sv), 16, 1024);
      const uint64_t ring_k = make_desc(smem_u32(smem + L::kRingOff), 16, 1024);            // streamed tiles as K-major B
      const uint64_t ring_mn = make_desc(smem_u32(smem + L::kRingOff), kSub * 128, 1024);   // the same tiles as MN-major B
      auto issue_scores = [&](int buf, int st) {
        const uint64_t b_q = desc_advance(ring_k, st * 2 * L::kSubBytes), b_do = desc_advance(b_q, L::kSubBytes);
        const uint32_t d_s = tmem_base + buf * 128, d_dp = d_s + 64;
        constexpr int kBlockA = kTile * 128, kBlockB = kSub * 128;
        // The two products alternate so that consecutive instructions never accumulate into the
        // same columns (a dependent chain runs at the pipeline latency, not at its throughput).
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_f16(d_s, desc_advance(dk_base, (kk / 4) * kBlockA + (kk % 4) * 32), desc_advance(b_q, (kk / 4) * kBlockB + (kk % 4) * 32),
                   idesc_s, kk > 0 ? 1u : 0u);
          umma_f16(d_dp, desc_advance(dv_base, (kk / 4) * kBlockA + (kk % 4) * 32), desc_advance(b_do, (kk / 4) * kBlockB + (kk % 4) * 32),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[buf]);
      };
      bool ok = mbar_wait(kv_full, 0, p.err, kErrAttnMma) && mbar_wait(&ring_full[0], 0, p.err, kErrAttnMma);
      if (ok) {
        tc_fence_after();
        issue_scores(0, 0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % L::kStages, buf = it & 1;
        if (it + 1 < n_it) {
          const int st1 = (it + 1) % L::kStages;
          if (!mbar_wait(&ring_full[st1], ((it + 1) / L::kStages) & 1, p.err, kErrAttnMma)) { ok = false; break; }
          tc_fence_after();
          stamp(it + 1, 1);  // MMA thread: operands of step it+1 landed, score MMAs issued
          issue_scores((it + 1) & 1, st1);
        }
        if (!mbar_wait(&pds_full[buf], (it >> 1) & 1, p.err, kErrAttnMma)) { ok = false; break; }
        tc_fence_after();
        stamp(it, 2);  // MMA thread: P / dS of step it ready, accumulate MMAs issued
        // A operands from tensor memory: group kk left P^T of its 16 queries in the first 8 columns of
        // its own score range (dS^T likewise in the dP range).  The next scores written to this
        // buffer are issued after these products by the same thread, so no extra barrier is needed.
        const uint32_t a_p = tmem_base + buf * 128, a_ds = a_p + 64;
        const uint64_t b_q = desc_advance(ring_mn, st * 2 * L::kSubBytes), b_do = desc_advance(b_q, L::kSubBytes);
#pragma unroll
        for (int kk = 0; kk < kSub / 16; ++kk) {
          umma_f16_ta(tmem_dv, a_p + kk * kCG, desc_advance(b_do, kk * 2048), idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
          umma_f16_ta(tmem_dk, a_ds + kk * kCG, desc_advance(b_q, kk * 2048), idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&ring_empty[st]);
        if (trace != nullptr) umma_commit(&acc_step[buf]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;    // which kCG columns of the 64-query sub-tile this group converts
    const int r = quarter * 32 + lane;  // key row within the tile
    const int key = key0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float* lse_row = p.lse + (static_cast<long long>(b) * p.H + h) * p.T;
    const float* delta_row = p.delta + (static_cast<long long>(b) * p.H + h) * p.T;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int buf = it & 1;
      const int q0 = (i0 + it) * kSub + grp * kCG;  // first query of this group's columns
      // Lane l holds the log2-scaled LSE and delta of query q0 + (l mod kCG); queries past the end
      // get +inf (P = 0).  Column values are fetched with shuffles below.
      const int q_lane = q0 + (lane % kCG);
      const float lse_lane = q_lane < p.T ? lse_row[q_lane] * 1.4426950408889634f : INFINITY;
      const float delta_lane = q_lane < p.T ? delta_row[q_lane] : 0.f;
      if (!warp_wait(&sdp_full[buf], (it >> 1) & 1, p.err, kErrAttnSoftmax)) { ok = false; break; }
      tc_fence_after();
      if (warp == 2 && lane == 0) stamp(it, 3);  // softmax warp: scores of step it complete
      float s[kCG], dp[kCG];
      tmem_ld16_nowait(tmem_base + buf * 128 + lane_off + grp * kCG, s);
      tmem_ld16_nowait(tmem_base + buf * 128 + lane_off + 64 + grp * kCG, dp);
      tmem_ld_wait();
      if (warp == 2 && lane == 0) stamp(it, 4);  // scores in registers
      __align__(16) uint32_t p_regs[kCG / 2];
      __align__(16) uint32_t ds_regs[kCG / 2];
      // Masking is needed only on tiles that touch the diagonal or the end of the sequence.
      const bool need_mask = (p.causal && (q0 < key0 + kTile)) || (key0 + kTile > p.T);
#pragma unroll
      for (int c8 = 0; c8 < kCG / 8; ++c8) {
        float l8[8], d8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          l8[e] = __shfl_sync(0xffffffffu, lse_lane, c8 * 8 + e);
          d8[e] = __shfl_sync(0xffffffffu, delta_lane, c8 * 8 + e);
        }
        float pv[8], dsv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = c8 * 8 + e;
          pv[e] = fast_exp2(fmaf(s[c], p.scale_log2, -l8[e]));
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (key >= p.T || (p.causal && key > q0 + c8 * 8 + e)) pv[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) dsv[e] = (pv[e] * p.scale) * (dp[c8 * 8 + e] - d8[e]);
        *reinterpret_cast<uint4*>(&p_regs[c8 * 4]) = pack8<T>(pv);
        *reinterpret_cast<uint4*>(&ds_regs[c8 * 4]) = pack8<T>(dsv);
      }
      tmem_st8(tmem_base + buf * 128 + lane_off + grp * kCG, p_regs);
      tmem_st8(tmem_base + buf * 128 + lane_off + 64 + grp * kCG, ds_regs);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[buf]);
      if (warp == 2 && lane == 0) stamp(it, 5);  // P / dS stored, hand-off signalled
    }
    if (ok && n_it > 0 && warp_wait(acc_done, 0, p.err, kErrAttnSoftmax)) {
      tc_fence_after();
      // Groups 0 and 1 write dV, groups 2 and 3 dK, each one 64-column block (D = 64: groups 0 and
      // 2 alone): stage this warp's 32 rows in the now idle V / K tile and store them.
      const int which = grp >> 1, block = grp & 1;
      if (block < D / 64) {
        uint8_t* dst = (which ? sk : sv) + block * (kTile * 128);
        const uint32_t src = (which ? tmem_dk : tmem_dv) + block * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          float o[32];
          tmem_ld32(src + lane_off + c * 32, o);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(dst + sw128_offset(r, c * 4 + q)) = pack8<T>(o + q * 8);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0 && key0 + quarter * 32 < p.T) {
          tma_store_3d(&map_dqkv, dst + quarter * 32 * 128, (which ? col_k : col_v) + block * 64, key0 + quarter * 32, b);
          tma_store_wait_all();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// dQ: one CTA per (batch, head, 128-query tile); streams 64-key sub-tiles of K and V.
//   S = Q K^T, dP = dO V^T (TMEM, 64 columns each, double buffered); one thread per query row
//   writes dS = P (dP - delta) * scale, packed to 16 bits, over its own score columns (TMEM), the A
//   operand of dQ += dS K (TMEM).
template <class T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_qkv128, const __grid_constant__ CUtensorMap map_qkv64,
                    const __grid_constant__ CUtensorMap map_do64, const __grid_constant__ CUtensorMap map_dqkv, FlashParams p) {
  using L = DqSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* ring_full = q_full + 1;
  uint64_t* ring_empty = ring_full + L::kStages;
  uint64_t* sdp_full = ring_empty + L::kStages;  // 2
  uint64_t* ds_full = sdp_full + 2;              // 2
  uint64_t* ds_free = ds_full + 2;               // 2
  uint64_t* acc_done = ds_free + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh - b * p.H;
  const int n_tiles = gridDim.y;
  const int qt = n_tiles - 1 - static_cast<int>(blockIdx.y);  // latest rows (most keys under the causal mask) first
  const int row0 = qt * kTile;
  const int last_q = min(p.T - 1, row0 + kTile - 1);
  const int n_it = p.causal ? (last_q / kSub + 1) : (p.T + kSub - 1) / kSub;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&ring_full[s], 1); mbar_init(&ring_empty[s], 1); }
    for (int w = 0; w < 2; ++w) { mbar_init(&sdp_full[w], 1); mbar_init(&ds_full[w], 4 * kBwdGroups); mbar_init(&ds_free[w], 1); }
    mbar_init(acc_done, 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base + 256;
  const int col_q = h * D, col_k = p.E + h * D, col_v = 2 * p.E + h * D;
  uint8_t* sq = smem + L::kBigOff;
  uint8_t* sdo = sq + L::kBigBytes;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * L::kBigBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_3d(sq + c * (kTile * 128), &map_qkv128, q_full, col_q + c * 64, row0, b);
        tma_load_3d(sdo + c * (kTile * 128), &map_do64, q_full, col_q + c * 64, row0, b);
        tma_load_3d(sdo + c * (kTile * 128) + kSub * 128, &map_do64, q_full, col_q + c * 64, row0 + kSub, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % L::kStages;
        if (!mbar_wait(&ring_empty[st], ((it / L::kStages) & 1) ^ 1, p.err, kErrAttnProducer)) break;
        mbar_expect_tx(&ring_full[st], 2 * L::kSubBytes);
        uint8_t* sk = smem + L::kRingOff + st * 2 * L::kSubBytes;
        uint8_t* sv = sk + L::kSubBytes;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_3d(sk + c * (kSub * 128), &map_qkv64, &ring_full[st], col_k + c * 64, it * kSub, b);
          tma_load_3d(sv + c * (kSub * 128), &map_qkv64, &ring_full[st], col_v + c * 64, it * kSub, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const bool bf = std::is_same<T, __nv_bfloat16>::value;
      const uint32_t idesc_s = make_idesc(bf, 0, 0, kTile, kSub);  // [128 queries x 64 keys], both K-major
      const uint32_t idesc_a = make_idesc(bf, 0, 1, kTile, D);     // [128 queries x D], K tile read MN-major
      const uint64_t dq_base = make_desc(smem_u32(sq), 16, 1024), ddo_base = make_desc(smem_u32(sdo), 16, 1024);
      const uint64_t ring_k = make_desc(smem_u32(smem + L::kRingOff), 16, 1024);            // streamed tiles as K-major B
      const uint64_t ring_mn = make_desc(smem_u32(smem + L::kRingOff), kSub * 128, 1024);   // the same tiles as MN-major B
      auto issue_scores = [&](int buf, int st) {
        const uint64_t b_k = desc_advance(ring_k, st * 2 * L::kSubBytes), b_v = desc_advance(b_k, L::kSubBytes);
        const uint32_t d_s = tmem_base + buf * 128, d_dp = d_s + 64;
        constexpr int kBlockA = kTile * 128, kBlockB = kSub * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {  // alternating accumulators, see the dK/dV kernel
          umma_f16(d_s, desc_advance(dq_base, (kk / 4) * kBlockA + (kk % 4) * 32), desc_advance(b_k, (kk / 4) * kBlockB + (kk % 4) * 32),
                   idesc_s, kk > 0 ? 1u : 0u);
          umma_f16(d_dp, desc_advance(ddo_base, (kk / 4) * kBlockA + (kk % 4) * 32), desc_advance(b_v, (kk / 4) * kBlockB + (kk % 4) * 32),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[buf]);
      };
      bool ok = mbar_wait(q_full, 0, p.err, kErrAttnMma) && mbar_wait(&ring_full[0], 0, p.err, kErrAttnMma);
      if (ok) {
        tc_fence_after();
        issue_scores(0, 0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % L::kStages, buf = it & 1;
        if (it + 1 < n_it) {
          const int st1 = (it + 1) % L::kStages;
          if (!mbar_wait(&ring_full[st1], ((it + 1) / L::kStages) & 1, p.err, kErrAttnMma)) { ok = false; break; }
          tc_fence_after();
          issue_scores((it + 1) & 1, st1);
        }
        if (!mbar_wait(&ds_full[buf], (it >> 1) & 1, p.err, kErrAttnMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_ds = tmem_base + buf * 128;  // dS of group kk in the first 8 columns of its score range
        const uint64_t b_k = desc_advance(ring_mn, st * 2 * L::kSubBytes);
#pragma unroll
        for (int kk = 0; kk < kSub / 16; ++kk)
          umma_f16_ta(tmem_dq, a_ds + kk * kCG, desc_advance(b_k, kk * 2048), idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&ring_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;  // which kCG columns of the 64-key sub-tile this group converts
    const int r = quarter * 32 + lane;
    const int q = row0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const long long vec_off = (static_cast<long long>(b) * p.H + h) * p.T + q;
    const float lse2 = q < p.T ? p.lse[vec_off] * 1.4426950408889634f : INFINITY;
    const float delta = q < p.T ? p.delta[vec_off] : 0.f;
    const int limit = p.causal ? min(q, p.T - 1) : p.T - 1;  // last visible key
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int buf = it & 1;
      const int k0 = it * kSub + grp * kCG;
      if (!warp_wait(&sdp_full[buf], (it >> 1) & 1, p.err, kErrAttnSoftmax)) { ok = false; break; }
      tc_fence_after();
      float s[kCG], dp[kCG];
      tmem_ld16_nowait(tmem_base + buf * 128 + lane_off + grp * kCG, s);
      tmem_ld16_nowait(tmem_base + buf * 128 + lane_off + 64 + grp * kCG, dp);
      tmem_ld_wait();
      __align__(16) uint32_t ds_regs[kCG / 2];
      const bool need_mask = (p.causal && (k0 + kCG - 1 > row0)) || (k0 + kCG > p.T);
#pragma unroll
      for (int c8 = 0; c8 < kCG / 8; ++c8) {
        float pv[8], dsv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) pv[e] = fast_exp2(fmaf(s[c8 * 8 + e], p.scale_log2, -lse2));
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (k0 + c8 * 8 + e > limit) pv[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) dsv[e] = (pv[e] * p.scale) * (dp[c8 * 8 + e] - delta);
        *reinterpret_cast<uint4*>(&ds_regs[c8 * 4]) = pack8<T>(dsv);
      }
      tmem_st8(tmem_base + buf * 128 + lane_off + grp * kCG, ds_regs);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[buf]);
    }
    if (ok && warp_wait(acc_done, 0, p.err, kErrAttnSoftmax)) {
      tc_fence_after();
      // Groups 0 and 1 each drain and store one 64-column block of dQ (group 0 alone when D = 64).
      if (grp < D / 64) {
#pragma unroll 1
        for (int c = grp * 2; c < grp * 2 + 2; ++c) {
          float o[32];
          tmem_ld32(tmem_dq + lane_off + c * 32, o);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            *reinterpret_cast<uint4*>(sq + grp * (kTile * 128) + sw128_offset(r, (c % 2) * 4 + e)) = pack8<T>(o + e * 8);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0 && row0 + quarter * 32 < p.T) {
          tma_store_3d(&map_dqkv, sq + grp * (kTile * 128) + quarter * 32 * 128, col_q + grp * 64, row0 + quarter * 32, b);
          tma_store_wait_all();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------- host side
struct AttnMaps {
  CUtensorMap qkv128;  // [B, T, 3E], box {64, 128, 1}
  CUtensorMap out32;   // [B, T, E],  box {64, 32, 1}
};

CUtensorMap make_map3(const Tensor& t, int cols, int T, int B, int box_rows, const char* what) {
  CUtensorMap m;
  const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[2] = {static_cast<uint64_t>(cols) * 2, static_cast<uint64_t>(cols) * 2 * static_cast<uint64_t>(T)};
  const uint32_t box[3] = {64, static_cast<uint32_t>(box_rows), 1};
  if (!tc05_encode_map(&m, t.dtype(), 3, t.data(), dims, strides, box))
    throw std::runtime_error(std::string("attention: cannot encode the tensor map of ") + what);
  return m;
}

template <class T, int D>
void launch_fwd(const Tensor& qkv, Tensor& out, Tensor& lse, int B, int Tn, int H, bool causal, float scale, cudaStream_t st) {
  using L = FwdSmem<D>;
  const int E = H * D;
  const CUtensorMap mq = make_map3(qkv, 3 * E, Tn, B, kTile, "qkv");
  const CUtensorMap mkv = make_map3(qkv, 3 * E, Tn, B, kKeys, "qkv");
  const CUtensorMap mo = make_map3(out, E, Tn, B, 32, "the output");
  FlashParams p{};
  p.B = B; p.H = H; p.T = Tn; p.E = E; p.causal = causal ? 1 : 0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse.data_as<float>();
  p.err = tc05_error_flag(qkv.device().index);
  static std::once_flag once;
  std::call_once(once, [] {
    OB_CUDA(cudaFuncSetAttribute(flash_fwd_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  });
  const int n_tiles = (Tn + kTile - 1) / kTile;
  dim3 grid(B * H, (n_tiles + 1) / 2);
  flash_fwd_kernel<T, D><<<grid, kFwdThreads, L::kTotal, st>>>(mq, mkv, mo, p);
  check_launch("flash_attention_forward");
}

template <class T, int D>
void launch_bwd(const Tensor& qkv, const Tensor& out, const Tensor& lse, const Tensor& dout, Tensor& dqkv, Tensor& delta, int B,
                int Tn, int H, bool causal, float scale, cudaStream_t st) {
  using LA = DkvSmem<D>;
  using LB = DqSmem<D>;
  const int E = H * D;
  const CUtensorMap m128 = make_map3(qkv, 3 * E, Tn, B, kTile, "qkv");
  const CUtensorMap m64 = make_map3(qkv, 3 * E, Tn, B, kSub, "qkv");
  const CUtensorMap mdo = make_map3(dout, E, Tn, B, kSub, "the output gradient");
  const CUtensorMap mdq = make_map3(dqkv, 3 * E, Tn, B, 32, "the qkv gradient");
  FlashParams p{};
  p.B = B; p.H = H; p.T = Tn; p.E = E; p.causal = causal ? 1 : 0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = const_cast<float*>(lse.data_as<float>());
  p.delta = delta.data_as<float>();
  p.err = tc05_error_flag(qkv.device().index);
  static std::once_flag once;
  std::call_once(once, [] {
    OB_CUDA(cudaFuncSetAttribute(flash_bwd_dkv_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, LA::kTotal));
    OB_CUDA(cudaFuncSetAttribute(flash_bwd_dq_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, LB::kTotal));
  });
  const long long rows = static_cast<long long>(B) * Tn * H;
  attn_delta_kernel<T><<<static_cast<unsigned>((rows * (D / 8) + 255) / 256), 256, 0, st>>>(dout.data_as<T>(), out.data_as<T>(),
                                                                                         delta.data_as<float>(), B, Tn, H, D);
  check_launch("attention_delta");
  const int n_tiles = (Tn + kTile - 1) / kTile;
  dim3 grid(B * H, n_tiles);
  static const bool want_trace = [] { const char* e = std::getenv("ORTHON_ATTENTION_TRACE"); return e != nullptr && e[0] == '1'; }();
  long long* trace_dev = nullptr;
  if (want_trace) {
    OB_CUDA(cudaMalloc(&trace_dev, 32 * 8 * sizeof(long long)));
    OB_CUDA(cudaMemsetAsync(trace_dev, 0, 32 * 8 * sizeof(long long), st));
    p.trace = trace_dev;
  }
  flash_bwd_dkv_kernel<T, D><<<grid, kBwdThreads, LA::kTotal, st>>>(m128, m64, mdo, mdq, p);
  check_launch("flash_attention_backward_dkv");
  if (want_trace) {
    long long host[32 * 8];
    OB_CUDA(cudaStreamSynchronize(st));
    OB_CUDA(cudaMemcpy(host, trace_dev, sizeof(host), cudaMemcpyDeviceToHost));
    OB_CUDA(cudaFree(trace_dev));
    p.trace = nullptr;
    long long t0 = 0;
    for (int k = 0; k < 32 * 8 && t0 == 0; ++k) t0 = host[k];
    for (int k = 0; k < 32 * 8; ++k) if (host[k] != 0 && host[k] < t0) t0 = host[k];
    std::fprintf(stderr, "attention dK/dV timeline of CTA (0,0), cycles since its first stamp\n"
                         "step  loads_issued  scores_issued  acc_issued  scores_seen  scores_in_regs  handoff\n");
    for (int it = 0; it < 32; ++it) {
      if (host[it * 8 + 3] == 0) continue;
      std::fprintf(stderr, "%4d", it);
      for (int slot = 0; slot < 7; ++slot) std::fprintf(stderr, " %13lld", host[it * 8 + slot] ? host[it * 8 + slot] - t0 : -1LL);
      std::fprintf(stderr, "\n");
    }
  }
  flash_bwd_dq_kernel<T, D><<<grid, kBwdThreads, LB::kTotal, st>>>(m128, m64, mdo, mdq, p);
  check_launch("flash_attention_backward_dq");
}

}  // namespace

// True when the fused kernels cover this problem (otherwise callers compose the op).
bool flash_attention_supported(const Tensor& qkv, int64_t heads) {
  if (!qkv.device().is_cuda() || qkv.ndim() != 3 || !qkv.is_contiguous()) return false;
  if (qkv.dtype() != DType::BF16 && qkv.dtype() != DType::F16) return false;
  const int64_t E = qkv.shape()[2] / 3;
  if (heads < 1 || E % heads != 0) return false;
  const int64_t D = E / heads;
  if (D != 64 && D != 128) return false;
  if ((reinterpret_cast<uintptr_t>(qkv.data()) & 15u) != 0) return false;
  if (qkv.shape()[1] < 1 || qkv.shape()[1] > 65535 * 64) return false;  // sequence tiles are the grid's y extent
  static const bool off = [] { const char* e = std::getenv("ORTHON_ATTENTION"); return e != nullptr && std::string(e) == "composed"; }();
  return !off;
}

// out[B, T, E] and lse[B, H, T] (float32) must be allocated by the caller.
void flash_attention_forward(const Tensor& qkv, int64_t heads, bool causal, double scale, Tensor& out, Tensor& lse, cudaStream_t st) {
  const int B = static_cast<int>(qkv.shape()[0]), Tn = static_cast<int>(qkv.shape()[1]);
  const int E = static_cast<int>(qkv.shape()[2] / 3), H = static_cast<int>(heads), D = E / H;
  DeviceGuard g(qkv.device().index);
  const float sc = static_cast<float>(scale);
  if (qkv.dtype() == DType::BF16) {
    if (D == 128) launch_fwd<__nv_bfloat16, 128>(qkv, out, lse, B, Tn, H, causal, sc, st);
    else launch_fwd<__nv_bfloat16, 64>(qkv, out, lse, B, Tn, H, causal, sc, st);
  } else {
    if (D == 128) launch_fwd<__half, 128>(qkv, out, lse, B, Tn, H, causal, sc, st);
    else launch_fwd<__half, 64>(qkv, out, lse, B, Tn, H, causal, sc, st);
  }
}

// dqkv[B, T, 3E] (fully overwritten) from qkv, the forward output and LSE, and dout[B, T, E];
// `delta` is float32 scratch of shape [B, H, T].
void flash_attention_backward(const Tensor& qkv, const Tensor& out, const Tensor& lse, const Tensor& dout, int64_t heads, bool causal,
                              double scale, Tensor& dqkv, Tensor& delta, cudaStream_t st) {
  const int B = static_cast<int>(qkv.shape()[0]), Tn = static_cast<int>(qkv.shape()[1]);
  const int E = static_cast<int>(qkv.shape()[2] / 3), H = static_cast<int>(heads), D = E / H;
  DeviceGuard g(qkv.device().index);
  const float sc = static_cast<float>(scale);
  if (qkv.dtype() == DType::BF16) {
    if (D == 128) launch_bwd<__nv_bfloat16, 128>(qkv, out, lse, dout, dqkv, delta, B, Tn, H, causal, sc, st);
    else launch_bwd<__nv_bfloat16, 64>(qkv, out, lse, dout, dqkv, delta, B, Tn, H, causal, sc, st);
  } else {
    if (D == 128) launch_bwd<__half, 128>(qkv, out, lse, dout, dqkv, delta, B, Tn, H, causal, sc, st);
    else launch_bwd<__half, 64>(qkv, out, lse, dout, dqkv, delta, B, Tn, H, causal, sc, st);
  }
}

// Entry points for the semantic-op layer: run on the device's current stream.
void flash_attention_forward_current(const Tensor& qkv, int64_t heads, bool causal, double scale, Tensor& out, Tensor& lse) {
  cudaStream_t st = static_cast<cudaStream_t>(Runtime::instance().cuda(qkv.device().index).current_stream());
  flash_attention_forward(qkv, heads, causal, scale, out, lse, st);
}
void flash_attention_backward_current(const Tensor& qkv, const Tensor& out, const Tensor& lse, const Tensor& dout, int64_t heads,
                                      bool causal, double scale, Tensor& dqkv, Tensor& delta) {
  cudaStream_t st = static_cast<cudaStream_t>(Runtime::instance().cuda(qkv.device().index).current_stream());
  flash_attention_backward(qkv, out, lse, dout, heads, causal, scale, dqkv, delta, st);
}

}  // namespace cu
}  // namespace ob

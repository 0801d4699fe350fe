// sm_100a fused training kernels that are bandwidth-bound: softmax / log-softmax (+bwd),
// fused softmax-cross-entropy with device-resident integer targets and 64-bit indexing,
// NLL, embedding gather / scatter-add, LayerNorm forward and backward (with the
// gamma/beta gradients), attention-score softmax with in-kernel causal masking, max pool.
//
// Replaces (reference project paths): src/backends/cuda/{softmax_kernels,
// cross_entropy_kernels,nll_loss_kernels,embedding_kernels,maxpool2d_kernels}.cu and the
// composed LayerNorm / attention-softmax of python/orthon/nn/layernorm.py:34-61 and
// python/orthon/functional/math.py:39-72.  Index errors never trap: out-of-range targets
// are clamped and counted in a device error word the host can poll.
#include "ob/cuda_common.cuh"
#include "ob/ops.h"

namespace ob {
namespace cu {

void sum_rows_f32(const float* in, float* out, int64_t outer, int64_t reduce, int64_t inner, float scale,
                  const Tensor& ref, cudaStream_t st);

namespace {

constexpr int kThreads = 256;

__device__ unsigned int g_index_errors = 0;  // count of clamped out-of-range indices

template <class I>
__device__ __forceinline__ int64_t checked_index(const I* idx, int64_t i, int64_t limit) {
  int64_t t = static_cast<int64_t>(idx[i]);
  if (t < 0 || t >= limit) {
    atomicAdd(&g_index_errors, 1u);
    t = t < 0 ? 0 : limit - 1;
  }
  return t;
}

// ------------------------------------------------------------------- softmax
// Rows of length `reduce` (inner == 1).  Online (max, sum) in one read, then a second
// read (an L1/L2 hit for rows of this size) writes the normalized values.
template <class T, bool LOG>
__global__ void softmax_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t reduce) {
  __shared__ float smem[32];
  const T* row = in + static_cast<int64_t>(blockIdx.x) * reduce;
  T* orow = out + static_cast<int64_t>(blockIdx.x) * reduce;
  float mx = -INFINITY;
  for (int64_t j = threadIdx.x; j < reduce; j += blockDim.x) mx = fmaxf(mx, to_f(row[j]));
  mx = block_max(mx, smem);
  float s = 0.f;
  for (int64_t j = threadIdx.x; j < reduce; j += blockDim.x) s += __expf(to_f(row[j]) - mx);
  s = block_sum(s, smem);
  const float ls = __logf(s), inv = 1.f / s;
  for (int64_t j = threadIdx.x; j < reduce; j += blockDim.x) {
    const float v = to_f(row[j]) - mx;
    orow[j] = from_f<T>(LOG ? v - ls : __expf(v) * inv);
  }
}

template <class T, bool LOG>
__global__ void softmax_inner_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t outer, int64_t reduce,
                                     int64_t inner) {
  const int64_t n = outer * inner;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t o = i / inner, k = i - o * inner;
    const T* base = in + o * reduce * inner + k;
    T* ob_ = out + o * reduce * inner + k;
    float mx = -INFINITY;
    for (int64_t r = 0; r < reduce; ++r) mx = fmaxf(mx, to_f(base[r * inner]));
    float s = 0.f;
    for (int64_t r = 0; r < reduce; ++r) s += __expf(to_f(base[r * inner]) - mx);
    const float ls = __logf(s), inv = 1.f / s;
    for (int64_t r = 0; r < reduce; ++r) {
      const float v = to_f(base[r * inner]) - mx;
      ob_[r * inner] = from_f<T>(LOG ? v - ls : __expf(v) * inv);
    }
  }
}

// dx = y*(g - sum(g*y))  (softmax)   or   g - exp(y)*sum(g)  (log-softmax); generic strides.
template <class T, bool LOG>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ g, T* __restrict__ out,
                                   int64_t reduce, int64_t inner) {
  __shared__ float smem[32];
  const int64_t o = blockIdx.x / inner, k = blockIdx.x - o * inner;
  const int64_t base = o * reduce * inner + k;
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < reduce; r += blockDim.x) {
    const float gv = to_f(g[base + r * inner]);
    acc += LOG ? gv : gv * to_f(y[base + r * inner]);
  }
  acc = block_sum(acc, smem);
  for (int64_t r = threadIdx.x; r < reduce; r += blockDim.x) {
    const float gv = to_f(g[base + r * inner]), yv = to_f(y[base + r * inner]);
    out[base + r * inner] = from_f<T>(LOG ? gv - __expf(yv) * acc : yv * (gv - acc));
  }
}

template <class T, bool LOG>
void k_softmax(OpCall& c) {
  const int64_t outer = c.i[0], reduce = c.i[1], inner = c.i[2];
  cudaStream_t st = stream_of(c);
  if (inner == 1) {
    if (outer > 2147483647LL) throw std::invalid_argument("softmax: too many rows");
    const int threads = reduce >= 1024 ? 256 : (reduce >= 256 ? 128 : 64);
    softmax_rows_kernel<T, LOG><<<static_cast<unsigned>(outer), threads, 0, st>>>(c.in[0].data_as<T>(), c.out[0].data_as<T>(), reduce);
  } else {
    softmax_inner_kernel<T, LOG><<<ew_grid(outer * inner, kThreads, sm_count_for(c.in[0])), kThreads, 0, st>>>(
        c.in[0].data_as<T>(), c.out[0].data_as<T>(), outer, reduce, inner);
  }
  check_launch("softmax");
}

template <class T, bool LOG>
void k_softmax_bwd(OpCall& c) {
  const int64_t outer = c.i[0], reduce = c.i[1], inner = c.i[2];
  if (outer * inner > 2147483647LL) throw std::invalid_argument("softmax backward: too many rows");
  const int threads = reduce >= 1024 ? 256 : (reduce >= 256 ? 128 : 64);
  softmax_bwd_kernel<T, LOG><<<static_cast<unsigned>(outer * inner), threads, 0, stream_of(c)>>>(
      c.in[0].data_as<T>(), c.in[1].data_as<T>(), c.out[0].data_as<T>(), reduce, inner);
  check_launch("softmax backward");
}

// ------------------------------------------------------------- cross entropy
template <class T, class I>
__global__ void xent_fwd_kernel(const T* __restrict__ logits, const I* __restrict__ targets, float* __restrict__ lse,
                                float* __restrict__ row_loss, int64_t C) {
  __shared__ float smem[32];
  const int64_t r = blockIdx.x;
  const T* row = logits + r * C;
  float mx = -INFINITY;
  constexpr int N = Pack<T>::N;
  const bool vec = (C % N == 0) && ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  if (vec) {
    for (int64_t j = threadIdx.x; j < C / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N);
#pragma unroll
      for (int k = 0; k < N; ++k) mx = fmaxf(mx, to_f(p.v[k]));
    }
  } else {
    for (int64_t j = threadIdx.x; j < C; j += blockDim.x) mx = fmaxf(mx, to_f(row[j]));
  }
  mx = block_max(mx, smem);
  float s = 0.f;
  if (vec) {
    for (int64_t j = threadIdx.x; j < C / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N);
#pragma unroll
      for (int k = 0; k < N; ++k) s += __expf(to_f(p.v[k]) - mx);
    }
  } else {
    for (int64_t j = threadIdx.x; j < C; j += blockDim.x) s += __expf(to_f(row[j]) - mx);
  }
  s = block_sum(s, smem);
  if (threadIdx.x == 0) {
    const float l = mx + __logf(s);
    lse[r] = l;
    row_loss[r] = l - to_f(row[checked_index(targets, r, C)]);
  }
}

template <class T, class I>
__global__ void xent_bwd_kernel(const T* __restrict__ logits, const I* __restrict__ targets,
                                const float* __restrict__ lse, const float* __restrict__ gscalar, T* __restrict__ out,
                                int64_t C, float inv_rows) {
  const int64_t r = blockIdx.x;
  const T* row = logits + r * C;
  T* orow = out + r * C;
  const float l = lse[r], g = gscalar[0] * inv_rows;
  const int64_t t = checked_index(targets, r, C);
  constexpr int N = Pack<T>::N;
  const bool vec = (C % N == 0) && ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0);
  if (vec) {
    for (int64_t j = threadIdx.x; j < C / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N), q;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const float sm = __expf(to_f(p.v[k]) - l);
        q.v[k] = from_f<T>((sm - ((j * N + k) == t ? 1.f : 0.f)) * g);
      }
      store_pack(orow + j * N, q);
    }
  } else {
    for (int64_t j = threadIdx.x; j < C; j += blockDim.x)
      orow[j] = from_f<T>((__expf(to_f(row[j]) - l) - (j == t ? 1.f : 0.f)) * g);
  }
}

template <class D>
__global__ void store_scalar_kernel(const float* __restrict__ v, D* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = from_f<D>(v[0]);
}

template <class S>
__global__ void load_scalar_kernel(const S* __restrict__ v, float* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = to_f(v[0]);
}

template <class T>
void k_xent(OpCall& c) {
  const Tensor& logits = c.in[0];
  const int64_t B = logits.shape()[0], C = logits.shape()[1];
  if (B > 2147483647LL) throw std::invalid_argument("cross_entropy: too many rows");
  cudaStream_t st = stream_of(c);
  ScratchLease lease(logits.device(), sizeof(float) * (B + 1), st);
  float* row_loss = static_cast<float*>(lease.data());
  float* mean = row_loss + B;
  float* lse = c.out[1].data_as<float>();
  if (c.in[1].dtype() == DType::I64)
    xent_fwd_kernel<T, int64_t><<<static_cast<unsigned>(B), kThreads, 0, st>>>(logits.data_as<T>(), c.in[1].data_as<int64_t>(), lse, row_loss, C);
  else
    xent_fwd_kernel<T, int32_t><<<static_cast<unsigned>(B), kThreads, 0, st>>>(logits.data_as<T>(), c.in[1].data_as<int32_t>(), lse, row_loss, C);
  sum_rows_f32(row_loss, mean, 1, B, 1, static_cast<float>(1.0 / static_cast<double>(B)), logits, st);
  if (c.out[0].dtype() == DType::F32) store_scalar_kernel<float><<<1, 32, 0, st>>>(mean, c.out[0].data_as<float>());
  else if (c.out[0].dtype() == DType::F16) store_scalar_kernel<__half><<<1, 32, 0, st>>>(mean, c.out[0].data_as<__half>());
  else store_scalar_kernel<__nv_bfloat16><<<1, 32, 0, st>>>(mean, c.out[0].data_as<__nv_bfloat16>());
  check_launch("cross_entropy");
}

template <class T>
void k_xent_bwd(OpCall& c) {
  const Tensor& logits = c.in[0];
  const int64_t B = logits.shape()[0], C = logits.shape()[1];
  cudaStream_t st = stream_of(c);
  const float inv = static_cast<float>(1.0 / static_cast<double>(B));
  // The upstream gradient may be float32 (loss of low-precision logits) or the logits dtype.
  ScratchLease lease(logits.device(), sizeof(float), st);
  float* gs = static_cast<float*>(lease.data());
  const Tensor& g = c.in[2];
  if (g.dtype() == DType::F32) load_scalar_kernel<float><<<1, 32, 0, st>>>(g.data_as<float>(), gs);
  else if (g.dtype() == DType::F16) load_scalar_kernel<__half><<<1, 32, 0, st>>>(g.data_as<__half>(), gs);
  else load_scalar_kernel<__nv_bfloat16><<<1, 32, 0, st>>>(g.data_as<__nv_bfloat16>(), gs);
  const float* lse = c.in[3].data_as<float>();
  if (c.in[1].dtype() == DType::I64)
    xent_bwd_kernel<T, int64_t><<<static_cast<unsigned>(B), kThreads, 0, st>>>(logits.data_as<T>(), c.in[1].data_as<int64_t>(), lse, gs, c.out[0].data_as<T>(), C, inv);
  else
    xent_bwd_kernel<T, int32_t><<<static_cast<unsigned>(B), kThreads, 0, st>>>(logits.data_as<T>(), c.in[1].data_as<int32_t>(), lse, gs, c.out[0].data_as<T>(), C, inv);
  check_launch("cross_entropy backward");
}

// ----------------------------------------------------------------------- NLL
template <class T, class I>
__global__ void nll_rows_kernel(const T* __restrict__ lp, const I* __restrict__ targets, float* __restrict__ rows,
                                T* __restrict__ out_none, int64_t N, int64_t C) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < N; i += stride) {
    const float v = -to_f(lp[i * C + checked_index(targets, i, C)]);
    if (out_none) out_none[i] = from_f<T>(v);
    else rows[i] = v;
  }
}

template <class T, class I>
__global__ void nll_bwd_kernel(const T* __restrict__ g, const I* __restrict__ targets, T* __restrict__ out, int64_t N,
                               int64_t C, int reduction) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < N; i += stride) {
    float gv = reduction == 0 ? to_f(g[i]) : to_f(g[0]);
    if (reduction == 1) gv /= static_cast<float>(N);
    out[i * C + checked_index(targets, i, C)] = from_f<T>(-gv);
  }
}

template <class T>
void k_nll(OpCall& c) {
  const Tensor& lp = c.in[0];
  const int64_t N = lp.shape()[0], C = lp.shape()[1];
  const int red = static_cast<int>(c.i[0]);
  cudaStream_t st = stream_of(c);
  const int grid = ew_grid(N, kThreads, sm_count_for(lp));
  const bool i64 = c.in[1].dtype() == DType::I64;
  if (red == 0) {
    if (i64) nll_rows_kernel<T, int64_t><<<grid, kThreads, 0, st>>>(lp.data_as<T>(), c.in[1].data_as<int64_t>(), nullptr, c.out[0].data_as<T>(), N, C);
    else nll_rows_kernel<T, int32_t><<<grid, kThreads, 0, st>>>(lp.data_as<T>(), c.in[1].data_as<int32_t>(), nullptr, c.out[0].data_as<T>(), N, C);
    check_launch("nll_loss");
    return;
  }
  ScratchLease lease(lp.device(), sizeof(float) * (N + 1), st);
  float* rows = static_cast<float*>(lease.data());
  if (i64) nll_rows_kernel<T, int64_t><<<grid, kThreads, 0, st>>>(lp.data_as<T>(), c.in[1].data_as<int64_t>(), rows, nullptr, N, C);
  else nll_rows_kernel<T, int32_t><<<grid, kThreads, 0, st>>>(lp.data_as<T>(), c.in[1].data_as<int32_t>(), rows, nullptr, N, C);
  sum_rows_f32(rows, rows + N, 1, N, 1, red == 1 ? static_cast<float>(1.0 / static_cast<double>(N)) : 1.f, lp, st);
  store_scalar_kernel<T><<<1, 32, 0, st>>>(rows + N, c.out[0].data_as<T>());
  check_launch("nll_loss");
}

template <class T>
void k_nll_bwd(OpCall& c) {
  Tensor& out = c.out[0];
  const int64_t N = out.shape()[0], C = out.shape()[1];
  cudaStream_t st = stream_of(c);
  OB_CUDA(cudaMemsetAsync(out.data(), 0, out.nbytes(), st));
  const int grid = ew_grid(N, kThreads, sm_count_for(out));
  if (c.in[1].dtype() == DType::I64)
    nll_bwd_kernel<T, int64_t><<<grid, kThreads, 0, st>>>(c.in[0].data_as<T>(), c.in[1].data_as<int64_t>(), out.data_as<T>(), N, C, static_cast<int>(c.i[0]));
  else
    nll_bwd_kernel<T, int32_t><<<grid, kThreads, 0, st>>>(c.in[0].data_as<T>(), c.in[1].data_as<int32_t>(), out.data_as<T>(), N, C, static_cast<int>(c.i[0]));
  check_launch("nll_loss backward");
}

// ----------------------------------------------------------------- embedding
template <class T, class I>
__global__ void embedding_fwd_kernel(const I* __restrict__ idx, const T* __restrict__ w, T* __restrict__ out,
                                     int64_t n, int64_t V, int64_t D) {
  // One warp per gathered row.
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  constexpr int N = Pack<T>::N;
  for (int64_t i = warp; i < n; i += nwarps) {
    const int64_t row = checked_index(idx, i, V);
    const T* src = w + row * D;
    T* dst = out + i * D;
    if (D % N == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
      for (int64_t j = lane; j < D / N; j += 32) store_pack(dst + j * N, load_pack(src + j * N));
    } else {
      for (int64_t j = lane; j < D; j += 32) dst[j] = src[j];
    }
  }
}

// Embedding backward, deterministic: dW[v] = sum over the positions i with idx[i] == v of g[i],
// added in increasing i.  Three steps, no floating-point atomics:
//   1. embedding_keys_kernel   validates the indices and writes (row, position) pairs;
//   2. embedding_sort_kernel   one thread block sorts the pairs by row with a stable LSD radix
//                              sort (8 bits per pass, as many passes as the vocabulary needs), so
//                              positions stay in increasing order inside a row;
//   3. embedding_segment_kernel one warp per pair; the warp whose pair starts a run of equal rows
//                              walks the run and adds the gradient rows in float32 registers, eight
//                              columns per lane at a time, then rounds once into dW.
// Rows that no position names keep the zeros written before step 3.
// (replaces the float32 atomicAdd scatter of the reference: src/backends/cuda/embedding_kernels.cu:65-148)
template <class I>
__global__ void embedding_keys_kernel(const I* __restrict__ idx, int* __restrict__ keys, int* __restrict__ pos, int64_t n, int64_t V) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    keys[i] = static_cast<int>(checked_index(idx, i, V));
    pos[i] = static_cast<int>(i);
  }
}

constexpr int kSortThreads = 1024;

// Stable: within a tile of 1024 pairs a thread's rank among equal digits is its count of
// lower-numbered threads with that digit (warp match + per-warp counts scanned in warp order),
// and tiles are processed in order with running per-digit bases.
__global__ void __launch_bounds__(kSortThreads) embedding_sort_kernel(int* __restrict__ keys_a, int* __restrict__ pos_a,
                                                                      int* __restrict__ keys_b, int* __restrict__ pos_b, int n, int passes) {
  __shared__ int base[256];
  __shared__ int warp_count[kSortThreads / 32][256];
  __shared__ int tile_total[256];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int *kin = keys_a, *pin = pos_a, *kout = keys_b, *pout = pos_b;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * 8;
    if (tid < 256) base[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kSortThreads) atomicAdd(&base[(kin[i] >> shift) & 255], 1);  // integer counts: order-free
    __syncthreads();
    if (tid == 0) {  // exclusive scan of 256 counts
      int run = 0;
      for (int d = 0; d < 256; ++d) { const int c = base[d]; base[d] = run; run += c; }
    }
    __syncthreads();
    for (int t0 = 0; t0 < n; t0 += kSortThreads) {
      for (int j = tid; j < (kSortThreads / 32) * 256; j += kSortThreads) (&warp_count[0][0])[j] = 0;
      __syncthreads();
      const int i = t0 + tid;
      const bool live = i < n;
      const int key = live ? kin[i] : 0, p = live ? pin[i] : 0;
      const int digit = (key >> shift) & 255;
      const unsigned active = __ballot_sync(0xFFFFFFFFu, live);
      int rank = 0;
      if (live) {
        const unsigned peers = __match_any_sync(active, digit);
        rank = __popc(peers & ((1u << lane) - 1u));
        if (rank == 0) warp_count[warp][digit] = __popc(peers);
      }
      __syncthreads();
      if (tid < 256) {  // per digit: offsets of the warps inside the tile, in warp order
        int run = 0;
        for (int w = 0; w < kSortThreads / 32; ++w) { const int c = warp_count[w][tid]; warp_count[w][tid] = run; run += c; }
        tile_total[tid] = run;
      }
      __syncthreads();
      if (live) {
        const int dst = base[digit] + warp_count[warp][digit] + rank;
        kout[dst] = key;
        pout[dst] = p;
      }
      __syncthreads();
      if (tid < 256) base[tid] += tile_total[tid];
      __syncthreads();
    }
    int* t = kin; kin = kout; kout = t;
    t = pin; pin = pout; pout = t;
    __syncthreads();
  }
}

template <class T>
__global__ void embedding_segment_kernel(const int* __restrict__ keys, const int* __restrict__ pos, const T* __restrict__ g,
                                         T* __restrict__ dw, int64_t n, int64_t D) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t j0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (j0 >= n) return;
  const int row = keys[j0];
  if (j0 > 0 && keys[j0 - 1] == row) return;  // not the head of its run
  int64_t j1 = j0 + 1;
  while (j1 < n && keys[j1] == row) ++j1;
  T* out = dw + static_cast<int64_t>(row) * D;
  const bool vec = (D % N == 0) && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(dw)) & 15u) == 0;
  if (vec) {
    for (int64_t c0 = static_cast<int64_t>(lane) * N; c0 < D; c0 += 32 * N) {
      float acc[N];
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = 0.f;
      for (int64_t j = j0; j < j1; ++j) {
        const Pack<T> p = load_pack(g + static_cast<int64_t>(pos[j]) * D + c0);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += to_f(p.v[k]);
      }
      Pack<T> q;
#pragma unroll
      for (int k = 0; k < N; ++k) q.v[k] = from_f<T>(acc[k]);
      store_pack(out + c0, q);
    }
  } else {
    for (int64_t c = lane; c < D; c += 32) {
      float acc = 0.f;
      for (int64_t j = j0; j < j1; ++j) acc += to_f(g[static_cast<int64_t>(pos[j]) * D + c]);
      out[c] = from_f<T>(acc);
    }
  }
}

template <class T>
void k_embedding(OpCall& c) {
  const Tensor &idx = c.in[0], &w = c.in[1];
  const int64_t n = idx.numel(), V = w.shape()[0], D = w.shape()[1];
  const int grid = ew_grid(n * 32, kThreads, sm_count_for(w));
  if (idx.dtype() == DType::I64)
    embedding_fwd_kernel<T, int64_t><<<grid, kThreads, 0, stream_of(c)>>>(idx.data_as<int64_t>(), w.data_as<T>(), c.out[0].data_as<T>(), n, V, D);
  else
    embedding_fwd_kernel<T, int32_t><<<grid, kThreads, 0, stream_of(c)>>>(idx.data_as<int32_t>(), w.data_as<T>(), c.out[0].data_as<T>(), n, V, D);
  check_launch("embedding");
}

template <class T>
void k_embedding_bwd(OpCall& c) {
  const Tensor &idx = c.in[0], &g = c.in[1];
  Tensor& dw = c.out[0];
  const int64_t n = idx.numel(), V = dw.shape()[0], D = dw.shape()[1];
  cudaStream_t st = stream_of(c);
  const int sms = sm_count_for(dw);
  OB_CUDA(cudaMemsetAsync(dw.data(), 0, dw.nbytes(), st));
  if (n == 0) return;
  if (n >= (int64_t(1) << 31) || V >= (int64_t(1) << 31)) throw std::invalid_argument("embedding backward: more than 2^31 - 1 indices or rows");
  // Two (row, position) buffers for the ping-pong passes of the sort.
  ScratchLease lease(dw.device(), sizeof(int) * 4 * static_cast<size_t>(n), st);
  int* keys_a = static_cast<int*>(lease.data());
  int *pos_a = keys_a + n, *keys_b = pos_a + n, *pos_b = keys_b + n;
  const int grid = ew_grid(n, kThreads, sms);
  if (idx.dtype() == DType::I64) embedding_keys_kernel<int64_t><<<grid, kThreads, 0, st>>>(idx.data_as<int64_t>(), keys_a, pos_a, n, V);
  else embedding_keys_kernel<int32_t><<<grid, kThreads, 0, st>>>(idx.data_as<int32_t>(), keys_a, pos_a, n, V);
  int passes = 1;
  while (passes < 4 && (V - 1) >> (8 * passes)) ++passes;
  embedding_sort_kernel<<<1, kSortThreads, 0, st>>>(keys_a, pos_a, keys_b, pos_b, static_cast<int>(n), passes);
  const int* keys = (passes & 1) ? keys_b : keys_a;
  const int* pos = (passes & 1) ? pos_b : pos_a;
  const int64_t warps_per_block = kThreads / 32;
  embedding_segment_kernel<T><<<static_cast<unsigned>((n + warps_per_block - 1) / warps_per_block), kThreads, 0, st>>>(
      keys, pos, g.data_as<T>(), dw.data_as<T>(), n, D);
  check_launch("embedding backward");
}

// ----------------------------------------------------------------- LayerNorm
// One block per row.  The row is re-read from L1 for the centered variance, so DRAM sees
// one read and one write per element.
template <class T>
__global__ void layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                     T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t D,
                                     float eps) {
  __shared__ float smem[32];
  const int64_t r = blockIdx.x;
  const T* row = x + r * D;
  T* orow = y + r * D;
  constexpr int N = Pack<T>::N;
  const bool vec = (D % N == 0) && ((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(orow)) & 15u) == 0 &&
                   (w == nullptr || (reinterpret_cast<uintptr_t>(w) & 15u) == 0) &&
                   (b == nullptr || (reinterpret_cast<uintptr_t>(b) & 15u) == 0);
  float s = 0.f;
  if (vec) {
    for (int64_t j = threadIdx.x; j < D / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N);
#pragma unroll
      for (int k = 0; k < N; ++k) s += to_f(p.v[k]);
    }
  } else {
    for (int64_t j = threadIdx.x; j < D; j += blockDim.x) s += to_f(row[j]);
  }
  const float m = block_sum(s, smem) / static_cast<float>(D);
  float v = 0.f;
  if (vec) {
    for (int64_t j = threadIdx.x; j < D / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { const float z = to_f(p.v[k]) - m; v += z * z; }
    }
  } else {
    for (int64_t j = threadIdx.x; j < D; j += blockDim.x) { const float z = to_f(row[j]) - m; v += z * z; }
  }
  const float rs = rsqrtf(block_sum(v, smem) / static_cast<float>(D) + eps);
  if (threadIdx.x == 0) { mean[r] = m; rstd[r] = rs; }
  if (vec) {
    for (int64_t j = threadIdx.x; j < D / N; j += blockDim.x) {
      Pack<T> p = load_pack(row + j * N), q;
      Pack<T> pw, pb;
      if (w) pw = load_pack(w + j * N);
      if (b) pb = load_pack(b + j * N);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float o = (to_f(p.v[k]) - m) * rs;
        if (w) o *= to_f(pw.v[k]);
        if (b) o += to_f(pb.v[k]);
        q.v[k] = from_f<T>(o);
      }
      store_pack(orow + j * N, q);
    }
  } else {
    for (int64_t j = threadIdx.x; j < D; j += blockDim.x) {
      float o = (to_f(row[j]) - m) * rs;
      if (w) o *= to_f(w[j]);
      if (b) o += to_f(b[j]);
      orow[j] = from_f<T>(o);
    }
  }
}

// Each block walks rows r = blockIdx.x, +gridDim.x, ...; per row it forms the two row sums,
// writes dx, and keeps per-column partial sums of g*xhat and g for the columns it owns
// (column j = threadIdx.x + k*blockDim.x).  Partials go to scratch [gridDim.x, 2, D].
template <class T, int MAXC>
__global__ void layernorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g,
                                     const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                                     float* __restrict__ partial, int64_t R, int64_t D, const T* __restrict__ addend) {
  __shared__ float smem[32];
  float dw_acc[MAXC], db_acc[MAXC];
#pragma unroll
  for (int k = 0; k < MAXC; ++k) dw_acc[k] = db_acc[k] = 0.f;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const T* xr = x + r * D;
    const T* gr = g + r * D;
    const float m = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int64_t j = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
      if (j < D) {
        const float xh = (to_f(xr[j]) - m) * rs;
        const float gv = to_f(gr[j]);
        const float gy = w ? gv * to_f(w[j]) : gv;
        s1 += gy;
        s2 += gy * xh;
        dw_acc[k] += gv * xh;
        db_acc[k] += gv;
      }
    }
    s1 = block_sum(s1, smem);
    s2 = block_sum(s2, smem);
    const float invD = 1.f / static_cast<float>(D);
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int64_t j = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
      if (j < D) {
        const float xh = (to_f(xr[j]) - m) * rs;
        const float gv = to_f(gr[j]);
        const float gy = w ? gv * to_f(w[j]) : gv;
        const float extra = addend ? to_f(addend[r * D + j]) : 0.f;
        dx[r * D + j] = from_f<T>(rs * (gy - s1 * invD - xh * s2 * invD) + extra);
      }
    }
  }
  if (partial) {
    float* pw = partial + static_cast<int64_t>(blockIdx.x) * 2 * D;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int64_t j = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
      if (j < D) { pw[j] = dw_acc[k]; pw[D + j] = db_acc[k]; }
    }
  }
}

template <class T>
__global__ void layernorm_bwd_finalize(const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db,
                                       int nblocks, int64_t D) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= D) return;
  float a = 0.f, b = 0.f;
  for (int i = 0; i < nblocks; ++i) {
    a += partial[static_cast<int64_t>(i) * 2 * D + j];
    b += partial[static_cast<int64_t>(i) * 2 * D + D + j];
  }
  if (dw) dw[j] = from_f<T>(a);
  if (db) db[j] = from_f<T>(b);
}

// ---- register-resident LayerNorm: every thread keeps its 16-byte packs of the row in
// registers between the statistics and the output pass, so each element is read once.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* smem /* 64 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) { smem[warp] = a; smem[32 + warp] = b; }
  __syncthreads();
  float ra = (threadIdx.x < nw) ? smem[threadIdx.x] : 0.f;
  float rb = (threadIdx.x < nw) ? smem[32 + threadIdx.x] : 0.f;
  if (warp == 0) {
    ra = warp_sum(ra);
    rb = warp_sum(rb);
    if (lane == 0) { smem[0] = ra; smem[32] = rb; }
  }
  __syncthreads();
  a = smem[0];
  b = smem[32];
}

template <class T, int CH>
__global__ void layernorm_fwd_fast(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                   T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t D,
                                   float eps) {
  constexpr int N = Pack<T>::N;
  __shared__ float smem[64];
  const int64_t r = blockIdx.x;
  const T* row = x + r * D;
  const int64_t npack = D / N;
  float v[CH][N];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
    if (p < npack) {
      Pack<T> pk = load_pack(row + p * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { v[c][k] = to_f(pk.v[k]); s += v[c][k]; }
    }
  }
  const float m = block_sum(s, smem) / static_cast<float>(D);
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
    if (p < npack) {
#pragma unroll
      for (int k = 0; k < N; ++k) { const float z = v[c][k] - m; q += z * z; }
    }
  }
  const float rs = rsqrtf(block_sum(q, smem) / static_cast<float>(D) + eps);
  if (threadIdx.x == 0) { mean[r] = m; rstd[r] = rs; }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
    if (p < npack) {
      Pack<T> pw, pb, out;
      if (w) pw = load_pack(w + p * N);
      if (b) pb = load_pack(b + p * N);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float o = (v[c][k] - m) * rs;
        if (w) o *= to_f(pw.v[k]);
        if (b) o += to_f(pb.v[k]);
        out.v[k] = from_f<T>(o);
      }
      store_pack(y + r * D + p * N, out);
    }
  }
}

template <class T, int CH>
__global__ void layernorm_bwd_fast(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g,
                                   const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                                   float* __restrict__ partial, int64_t R, int64_t D, const T* __restrict__ addend) {
  constexpr int N = Pack<T>::N;
  __shared__ float smem[64];
  const int64_t npack = D / N;
  float wv[CH][N], dw_acc[CH][N], db_acc[CH][N];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
    Pack<T> pw;
    if (w && p < npack) pw = load_pack(w + p * N);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      wv[c][k] = (w && p < npack) ? to_f(pw.v[k]) : 1.f;
      dw_acc[c][k] = db_acc[c][k] = 0.f;
    }
  }
  // The loads of the next row are issued before the current row's two block-wide sums, so a
  // block always has a row of DRAM requests in flight while it synchronises.  The row is kept as
  // loaded (16-bit packs) and the normalised values are formed twice rather than held in float32
  // registers: that keeps the block small enough for several per SM.
  Pack<T> cx[CH], cg[CH], ca[CH], nx[CH], ng[CH], na[CH];
  float cm = 0.f, crs = 0.f, nm = 0.f, nrs = 0.f;
  auto fetch = [&](int64_t r, Pack<T>* fx, Pack<T>* fg, Pack<T>* fa, float& fm, float& frs) {
    fm = mean[r]; frs = rstd[r];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
      if (p < npack) {
        fx[c] = load_pack(x + r * D + p * N);
        fg[c] = load_pack(g + r * D + p * N);
        if (addend) fa[c] = load_pack(addend + r * D + p * N);
      }
    }
  };
  constexpr bool kAhead = CH == 1;   // wider rows would pay for the second set of packs with their occupancy
  if (kAhead && static_cast<int64_t>(blockIdx.x) < R) fetch(blockIdx.x, cx, cg, ca, cm, crs);
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const bool more = kAhead && r + gridDim.x < R;
    if (more) fetch(r + gridDim.x, nx, ng, na, nm, nrs);
    if (!kAhead) fetch(r, cx, cg, ca, cm, crs);
    const float m = cm, rs = crs;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
      if (p < npack) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float gv = to_f(cg[c].v[k]);
          const float xh = (to_f(cx[c].v[k]) - m) * rs;
          const float gy = gv * wv[c][k];
          s1 += gy;
          s2 += gy * xh;
          dw_acc[c][k] += gv * xh;
          db_acc[c][k] += gv;
        }
      }
    }
    block_sum2(s1, s2, smem);
    const float invD = 1.f / static_cast<float>(D);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
      if (p < npack) {
        Pack<T> out;
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float xh = (to_f(cx[c].v[k]) - m) * rs;
          const float gy = to_f(cg[c].v[k]) * wv[c][k];
          out.v[k] = from_f<T>(rs * (gy - s1 * invD - xh * s2 * invD) + (addend ? to_f(ca[c].v[k]) : 0.f));
        }
        store_pack(dx + r * D + p * N, out);
      }
    }
    if (more) {
#pragma unroll
      for (int c = 0; c < CH; ++c) { cx[c] = nx[c]; cg[c] = ng[c]; ca[c] = na[c]; }
      cm = nm; crs = nrs;
    }
  }
  if (partial) {
    float* pw_ = partial + static_cast<int64_t>(blockIdx.x) * 2 * D;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int64_t p = static_cast<int64_t>(c) * blockDim.x + threadIdx.x;
      if (p < npack) {
#pragma unroll
        for (int k = 0; k < N; ++k) { pw_[p * N + k] = dw_acc[c][k]; pw_[D + p * N + k] = db_acc[c][k]; }
      }
    }
  }
}

// Column sums of the per-block partials: block (32, 32), one 32-column strip per block; the 32
// row groups keep enough loads in flight to hide DRAM latency, then a fixed-order sum.
template <class T>
__global__ void layernorm_bwd_finalize_fast(const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db,
                                            int nblocks, int64_t D) {
  __shared__ float ta[32][33], tb[32][33];
  const int64_t j = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (j < D) {
#pragma unroll 4
    for (int i = threadIdx.y; i < nblocks; i += 32) {
      a += partial[static_cast<int64_t>(i) * 2 * D + j];
      b += partial[static_cast<int64_t>(i) * 2 * D + D + j];
    }
  }
  ta[threadIdx.y][threadIdx.x] = a;
  tb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && j < D) {
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { sa += ta[i][threadIdx.x]; sb += tb[i][threadIdx.x]; }
    if (dw) dw[j] = from_f<T>(sa);
    if (db) db[j] = from_f<T>(sb);
  }
}

// First stage for many partial rows: group g adds its share of the rows (fixed order) into
// out[g][2][D], so that the final pass above reads a few dozen rows instead of thousands.
// grid = (ceil(D / 32), groups), block = (32, 32).
__global__ void layernorm_bwd_group_partials(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int64_t D) {
  __shared__ float ta[32][33], tb[32][33];
  const int64_t j = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  const int per = (nblocks + gridDim.y - 1) / gridDim.y;
  const int begin = blockIdx.y * per, end = min(nblocks, begin + per);
  float a = 0.f, b = 0.f;
  if (j < D) {
#pragma unroll 4
    for (int i = begin + threadIdx.y; i < end; i += 32) {
      a += partial[static_cast<int64_t>(i) * 2 * D + j];
      b += partial[static_cast<int64_t>(i) * 2 * D + D + j];
    }
  }
  ta[threadIdx.y][threadIdx.x] = a;
  tb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && j < D) {
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { sa += ta[i][threadIdx.x]; sb += tb[i][threadIdx.x]; }
    out[static_cast<int64_t>(blockIdx.y) * 2 * D + j] = sa;
    out[static_cast<int64_t>(blockIdx.y) * 2 * D + D + j] = sb;
  }
}

template <class T>
bool ln_fast_ok(const OpCall& c, int64_t D, int* threads, int* chunks) {
  constexpr int N = Pack<T>::N;
  if (D % N != 0) return false;
  const int64_t npack = D / N;
  if (npack > 256 * 4) return false;
  for (int i = 0; i < 5; ++i)
    if (c.in[i].defined() && !aligned16(c.in[i].data())) return false;
  if (!aligned16(c.out[0].data())) return false;
  int ch = static_cast<int>((npack + 255) / 256);
  if (ch == 3) ch = 4;
  int th = static_cast<int>((npack + ch - 1) / ch);
  th = ((th + 31) / 32) * 32;
  *threads = th;
  *chunks = ch;
  return true;
}

// One warp per row: CH packs per lane (pack index c * 32 + lane, so every load is a full line),
// statistics by shuffles only.  Four rows per block.  Requires D == CH * 32 * Pack<T>::N.
template <class T, int CH>
__global__ void __launch_bounds__(128) layernorm_fwd_warp(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                          T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd,
                                                          int64_t R, float eps) {
  constexpr int N = Pack<T>::N;
  constexpr int D = CH * 32 * N;
  const int lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (r >= R) return;
  const T* row = x + r * D;
  float v[CH][N];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const Pack<T> pk = load_pack(row + (c * 32 + lane) * N);
#pragma unroll
    for (int k = 0; k < N; ++k) { v[c][k] = to_f(pk.v[k]); s += v[c][k]; }
  }
  const float m = warp_sum(s) * (1.f / D);
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int k = 0; k < N; ++k) { const float z = v[c][k] - m; q += z * z; }
  const float rs = rsqrtf(warp_sum(q) * (1.f / D) + eps);
  if (lane == 0) { mean[r] = m; rstd[r] = rs; }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int off = (c * 32 + lane) * N;
    Pack<T> pw, pb, out;
    if (w) pw = load_pack(w + off);
    if (b) pb = load_pack(b + off);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float o = (v[c][k] - m) * rs;
      if (w) o *= to_f(pw.v[k]);
      if (b) o += to_f(pb.v[k]);
      out.v[k] = from_f<T>(o);
    }
    store_pack(y + r * D + off, out);
  }
}

template <class T>
bool layernorm_fwd_warp_launch(const T* x, const T* w, const T* b, T* y, float* mean, float* rstd, int64_t R, int64_t D, float eps,
                               cudaStream_t st) {
  constexpr int N = Pack<T>::N;
  if (D % (32 * N) != 0) return false;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b)) & 15u)
    return false;
  const unsigned grid = static_cast<unsigned>((R + 3) / 4);
  switch (D / (32 * N)) {
    case 1: layernorm_fwd_warp<T, 1><<<grid, 128, 0, st>>>(x, w, b, y, mean, rstd, R, eps); return true;
    case 2: layernorm_fwd_warp<T, 2><<<grid, 128, 0, st>>>(x, w, b, y, mean, rstd, R, eps); return true;
    case 4: layernorm_fwd_warp<T, 4><<<grid, 128, 0, st>>>(x, w, b, y, mean, rstd, R, eps); return true;
    case 8: layernorm_fwd_warp<T, 8><<<grid, 128, 0, st>>>(x, w, b, y, mean, rstd, R, eps); return true;
    default: return false;
  }
}

template <class T>
void k_layernorm(OpCall& c) {
  const Tensor& x = c.in[0];
  const int64_t R = x.shape()[0], D = x.shape()[1];
  if (R > 2147483647LL) throw std::invalid_argument("layer_norm: too many rows");
  const T* fw = c.in[1].defined() ? c.in[1].data_as<T>() : nullptr;
  const T* fb = c.in[2].defined() ? c.in[2].data_as<T>() : nullptr;
  if (x.is_contiguous() && c.out[0].is_contiguous() &&
      layernorm_fwd_warp_launch<T>(x.data_as<T>(), fw, fb, c.out[0].data_as<T>(), c.out[1].data_as<float>(), c.out[2].data_as<float>(), R,
                                   D, static_cast<float>(c.f[0]), stream_of(c))) {
    check_launch("layer_norm");
    return;
  }
  int fth = 0, fch = 0;
  if (ln_fast_ok<T>(c, D, &fth, &fch)) {
    cudaStream_t st = stream_of(c);
    float* pm = c.out[1].data_as<float>();
    float* pr = c.out[2].data_as<float>();
    const float eps = static_cast<float>(c.f[0]);
    if (fch == 1) layernorm_fwd_fast<T, 1><<<static_cast<unsigned>(R), fth, 0, st>>>(x.data_as<T>(), fw, fb, c.out[0].data_as<T>(), pm, pr, D, eps);
    else if (fch == 2) layernorm_fwd_fast<T, 2><<<static_cast<unsigned>(R), fth, 0, st>>>(x.data_as<T>(), fw, fb, c.out[0].data_as<T>(), pm, pr, D, eps);
    else layernorm_fwd_fast<T, 4><<<static_cast<unsigned>(R), fth, 0, st>>>(x.data_as<T>(), fw, fb, c.out[0].data_as<T>(), pm, pr, D, eps);
    check_launch("layer_norm");
    return;
  }
  const int per = Pack<T>::N;
  int threads = static_cast<int>(std::min<int64_t>(256, std::max<int64_t>(32, ((D / per + 31) / 32) * 32)));
  layernorm_fwd_kernel<T><<<static_cast<unsigned>(R), threads, 0, stream_of(c)>>>(
      x.data_as<T>(), c.in[1].defined() ? c.in[1].data_as<T>() : nullptr, c.in[2].defined() ? c.in[2].data_as<T>() : nullptr,
      c.out[0].data_as<T>(), c.out[1].data_as<float>(), c.out[2].data_as<float>(), D, static_cast<float>(c.f[0]));
  check_launch("layer_norm");
}

constexpr int kLnGroups = 32;  // row groups of the two-stage reduction of the LayerNorm parameter-gradient partials

template <class T>
void k_layernorm_bwd(OpCall& c) {
  const Tensor& x = c.in[0];
  const int64_t R = x.shape()[0], D = x.shape()[1];
  cudaStream_t st = stream_of(c);
  const int sms = sm_count_for(x);
  const int threads = 256;
  if (D > 256 * 32) throw std::invalid_argument("layer_norm backward: normalized size above 8192 is not supported on CUDA");
  int fth = 0, fch = 0;
  const bool fast = ln_fast_ok<T>(c, D, &fth, &fch);
  // Rows are walked by persistent blocks.  Narrow rows give small blocks (64 threads for 512
  // columns), so more of them are needed per SM to keep enough loads in flight: up to 1024
  // resident threads per SM (64 registers each), at most 16 blocks.
  int per_sm = fast ? std::max(4, std::min(16, 1024 / std::max(fth, 1))) : 4;
  if (fast) {
    // Never more blocks than can be resident: the rows are dealt out statically.
    int resident = per_sm;
    const cudaError_t e = fch == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, layernorm_bwd_fast<T, 1>, fth, 0)
                          : fch == 2 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, layernorm_bwd_fast<T, 2>, fth, 0)
                                     : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, layernorm_bwd_fast<T, 4>, fth, 0);
    if (e == cudaSuccess && resident >= 1) per_sm = std::min(per_sm, resident);
    else (void)cudaGetLastError();
  }
  const int nblocks = static_cast<int>(std::min<int64_t>(R, static_cast<int64_t>(sms) * per_sm));
  const bool need_params = c.out[1].defined() || c.out[2].defined();
  ScratchLease lease;
  float* partial = nullptr;
  if (need_params) {
    lease = ScratchLease(x.device(), sizeof(float) * (nblocks + kLnGroups) * 2 * D, st);
    partial = static_cast<float*>(lease.data());
  }
  const T* pw = c.in[1].defined() ? c.in[1].data_as<T>() : nullptr;
  const T* padd = c.in[5].defined() ? c.in[5].data_as<T>() : nullptr;   // running gradient of the input, added to dx
  if (fast) {
    const T* px = x.data_as<T>();
    const T* pg = c.in[2].data_as<T>();
    const float* pmn = c.in[3].data_as<float>();
    const float* prs = c.in[4].data_as<float>();
    T* pdx = c.out[0].data_as<T>();
    if (fch == 1) layernorm_bwd_fast<T, 1><<<nblocks, fth, 0, st>>>(px, pw, pg, pmn, prs, pdx, partial, R, D, padd);
    else if (fch == 2) layernorm_bwd_fast<T, 2><<<nblocks, fth, 0, st>>>(px, pw, pg, pmn, prs, pdx, partial, R, D, padd);
    else layernorm_bwd_fast<T, 4><<<nblocks, fth, 0, st>>>(px, pw, pg, pmn, prs, pdx, partial, R, D, padd);
    if (need_params) {
      const float* rows = partial;
      int nrows = nblocks;
      if (nblocks > 1024) {  // narrow rows: thousands of partial rows, reduce them in two stages
        float* grouped = partial + static_cast<int64_t>(nblocks) * 2 * D;
        layernorm_bwd_group_partials<<<dim3(static_cast<unsigned>((D + 31) / 32), kLnGroups), dim3(32, 32), 0, st>>>(partial, grouped, nblocks, D);
        rows = grouped;
        nrows = kLnGroups;
      }
      layernorm_bwd_finalize_fast<T><<<static_cast<unsigned>((D + 31) / 32), dim3(32, 32), 0, st>>>(
          rows, c.out[1].defined() ? c.out[1].data_as<T>() : nullptr, c.out[2].defined() ? c.out[2].data_as<T>() : nullptr, nrows, D);
    }
    check_launch("layer_norm backward");
    return;
  }
  const int cols = static_cast<int>((D + threads - 1) / threads);
#define LN_BWD(MAXC)                                                                                          \
  layernorm_bwd_kernel<T, MAXC><<<nblocks, threads, 0, st>>>(x.data_as<T>(), pw, c.in[2].data_as<T>(),           \
                                                             c.in[3].data_as<float>(), c.in[4].data_as<float>(), \
                                                             c.out[0].data_as<T>(), partial, R, D, padd)
  if (cols <= 2) LN_BWD(2);
  else if (cols <= 4) LN_BWD(4);
  else if (cols <= 8) LN_BWD(8);
  else if (cols <= 16) LN_BWD(16);
  else LN_BWD(32);
#undef LN_BWD
  if (need_params)
    layernorm_bwd_finalize<T><<<static_cast<unsigned>((D + 255) / 256), 256, 0, st>>>(
        partial, c.out[1].defined() ? c.out[1].data_as<T>() : nullptr, c.out[2].defined() ? c.out[2].data_as<T>() : nullptr, nblocks, D);
  check_launch("layer_norm backward");
}

// --------------------------------------------------------- attention softmax
// One warp per score row.  probs = softmax(scale*s + mask) with column j masked out when
// causal and j > i + (Tk - Tq).
template <class T>
__global__ void attn_softmax_kernel(const T* __restrict__ s, const T* __restrict__ mask, T* __restrict__ p,
                                    int64_t rows, int64_t Tq, int64_t Tk, float scale, int causal) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const int64_t i = row % Tq;
  const int64_t limit = causal ? min(Tk, i + (Tk - Tq) + 1) : Tk;  // columns [0, limit) are visible
  const T* sr = s + row * Tk;
  const T* mr = mask ? mask + i * Tk : nullptr;
  T* pr = p + row * Tk;
  float mx = -INFINITY;
  for (int64_t j = lane; j < limit; j += 32) {
    float v = to_f(sr[j]) * scale;
    if (mr) v += to_f(mr[j]);
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int64_t j = lane; j < limit; j += 32) {
    float v = to_f(sr[j]) * scale;
    if (mr) v += to_f(mr[j]);
    sum += __expf(v - mx);
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int64_t j = lane; j < Tk; j += 32) {
    float o = 0.f;
    if (j < limit) {
      float v = to_f(sr[j]) * scale;
      if (mr) v += to_f(mr[j]);
      o = __expf(v - mx) * inv;
    }
    pr[j] = from_f<T>(o);
  }
}

template <class T>
__global__ void attn_softmax_bwd_kernel(const T* __restrict__ p, const T* __restrict__ g, T* __restrict__ out,
                                        int64_t rows, int64_t Tk, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const T* pr = p + row * Tk;
  const T* gr = g + row * Tk;
  T* orow = out + row * Tk;
  float dot = 0.f;
  for (int64_t j = lane; j < Tk; j += 32) dot += to_f(pr[j]) * to_f(gr[j]);
  dot = warp_sum(dot);
  for (int64_t j = lane; j < Tk; j += 32) orow[j] = from_f<T>(to_f(pr[j]) * (to_f(gr[j]) - dot) * scale);
}

template <class T>
void k_attn_softmax(OpCall& c) {
  const Tensor& s = c.in[0];
  const int64_t rows = s.shape()[0] * s.shape()[1], Tq = s.shape()[1], Tk = s.shape()[2];
  const int64_t blocks = (rows * 32 + 127) / 128;
  if (blocks > 2147483647LL) throw std::invalid_argument("attention softmax: too many rows");
  attn_softmax_kernel<T><<<static_cast<unsigned>(blocks), 128, 0, stream_of(c)>>>(
      s.data_as<T>(), c.in[1].defined() ? c.in[1].data_as<T>() : nullptr, c.out[0].data_as<T>(), rows, Tq, Tk,
      static_cast<float>(c.f[0]), static_cast<int>(c.i[0]));
  check_launch("attention softmax");
}

template <class T>
void k_attn_softmax_bwd(OpCall& c) {
  const Tensor& p = c.in[0];
  const int64_t rows = p.shape()[0] * p.shape()[1], Tk = p.shape()[2];
  const int64_t blocks = (rows * 32 + 127) / 128;
  attn_softmax_bwd_kernel<T><<<static_cast<unsigned>(blocks), 128, 0, stream_of(c)>>>(
      p.data_as<T>(), c.in[1].data_as<T>(), c.out[0].data_as<T>(), rows, Tk, static_cast<float>(c.f[0]));
  check_launch("attention softmax backward");
}

// ------------------------------------------------------------------- maxpool
struct PoolGeom { int kh, kw, sh, sw, ph, pw; int64_t H, W, OH, OW; };

template <class T>
__device__ __forceinline__ int64_t pool_argmax(const T* plane, const PoolGeom& g, int64_t oh, int64_t ow) {
  int64_t best = -1;
  float bv = 0.f;
  for (int r = 0; r < g.kh; ++r) {
    const int64_t ih = oh * g.sh - g.ph + r;
    if (ih < 0 || ih >= g.H) continue;
    for (int s = 0; s < g.kw; ++s) {
      const int64_t iw = ow * g.sw - g.pw + s;
      if (iw < 0 || iw >= g.W) continue;
      const float v = to_f(plane[ih * g.W + iw]);
      if (best < 0) { best = ih * g.W + iw; bv = v; continue; }
      const bool vn = v != v, bn = bv != bv;
      if ((bn && !vn) || (!vn && !bn && v > bv)) { best = ih * g.W + iw; bv = v; }
    }
  }
  return best;
}

template <class T>
__global__ void maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t planes, PoolGeom g) {
  const int64_t n = planes * g.OH * g.OW;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t ow = i % g.OW, oh = (i / g.OW) % g.OH, p = i / (g.OW * g.OH);
    const T* plane = x + p * g.H * g.W;
    const int64_t a = pool_argmax(plane, g, oh, ow);
    out[i] = a < 0 ? from_f<T>(-INFINITY) : plane[a];
  }
}

// One thread per input pixel: re-derives the argmax of every window that covers it, so the
// result is deterministic and needs no atomics.
template <class T>
__global__ void maxpool_bwd_kernel(const T* __restrict__ x, const T* __restrict__ grad, T* __restrict__ dx,
                                   int64_t planes, PoolGeom g) {
  const int64_t n = planes * g.H * g.W;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t iw = i % g.W, ih = (i / g.W) % g.H, p = i / (g.W * g.H);
    const T* plane = x + p * g.H * g.W;
    const T* gp = grad + p * g.OH * g.OW;
    float acc = 0.f;
    int64_t oh_lo = (ih + g.ph - g.kh + g.sh) / g.sh;  // ceil((ih+ph-kh+1)/sh)
    if (ih + g.ph - g.kh + 1 <= 0) oh_lo = 0;
    int64_t oh_hi = (ih + g.ph) / g.sh;
    if (oh_hi >= g.OH) oh_hi = g.OH - 1;
    int64_t ow_lo = (iw + g.pw - g.kw + g.sw) / g.sw;
    if (iw + g.pw - g.kw + 1 <= 0) ow_lo = 0;
    int64_t ow_hi = (iw + g.pw) / g.sw;
    if (ow_hi >= g.OW) ow_hi = g.OW - 1;
    for (int64_t oh = oh_lo; oh <= oh_hi; ++oh)
      for (int64_t ow = ow_lo; ow <= ow_hi; ++ow)
        if (pool_argmax(plane, g, oh, ow) == ih * g.W + iw) acc += to_f(gp[oh * g.OW + ow]);
    dx[i] = from_f<T>(acc);
  }
}

PoolGeom pool_geom(const OpCall& c, const Tensor& x, int64_t OH, int64_t OW) {
  PoolGeom g;
  g.kh = static_cast<int>(c.i[0]); g.kw = static_cast<int>(c.i[1]); g.sh = static_cast<int>(c.i[2]);
  g.sw = static_cast<int>(c.i[3]); g.ph = static_cast<int>(c.i[4]); g.pw = static_cast<int>(c.i[5]);
  g.H = x.shape()[2]; g.W = x.shape()[3]; g.OH = OH; g.OW = OW;
  return g;
}

template <class T>
void k_maxpool(OpCall& c) {
  const Tensor& x = c.in[0];
  Tensor& out = c.out[0];
  const PoolGeom g = pool_geom(c, x, out.shape()[2], out.shape()[3]);
  const int64_t planes = x.shape()[0] * x.shape()[1];
  maxpool_fwd_kernel<T><<<ew_grid(out.numel(), kThreads, sm_count_for(x)), kThreads, 0, stream_of(c)>>>(
      x.data_as<T>(), out.data_as<T>(), planes, g);
  check_launch("maxpool2d");
}

template <class T>
void k_maxpool_bwd(OpCall& c) {
  const Tensor &x = c.in[0], &grad = c.in[1];
  const PoolGeom g = pool_geom(c, x, grad.shape()[2], grad.shape()[3]);
  const int64_t planes = x.shape()[0] * x.shape()[1];
  maxpool_bwd_kernel<T><<<ew_grid(x.numel(), kThreads, sm_count_for(x)), kThreads, 0, stream_of(c)>>>(
      x.data_as<T>(), grad.data_as<T>(), c.out[0].data_as<T>(), planes, g);
  check_launch("maxpool2d backward");
}

template <class T> void k_softmax_f(OpCall& c) { k_softmax<T, false>(c); }
template <class T> void k_log_softmax_f(OpCall& c) { k_softmax<T, true>(c); }
template <class T> void k_softmax_b(OpCall& c) { k_softmax_bwd<T, false>(c); }
template <class T> void k_log_softmax_b(OpCall& c) { k_softmax_bwd<T, true>(c); }

}  // namespace

// Number of out-of-range indices clamped by kernels since the last call (and reset).
unsigned int take_index_errors() {
  unsigned int host = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&host, g_index_errors, sizeof(host)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaMemcpyToSymbol(g_index_errors, &zero, sizeof(zero));
  return host;
}

void register_cuda_nn(KernelRegistry& r) {
  const uint8_t packed = kContiguous | kEmpty;
#define REG3(OP, FN, NAME)                                                                                      \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, kMaskF32, packed, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::F16), packed, Capability::None}, FN<__half>, NAME "_f16"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::BF16), packed, Capability::Bf16}, FN<__nv_bfloat16>, NAME "_bf16");
  REG3(Softmax, k_softmax_f, "sm100_softmax") REG3(LogSoftmax, k_log_softmax_f, "sm100_log_softmax")
  REG3(SoftmaxBackward, k_softmax_b, "sm100_softmax_backward")
  REG3(LogSoftmaxBackward, k_log_softmax_b, "sm100_log_softmax_backward")
  REG3(CrossEntropy, k_xent, "sm100_softmax_xent") REG3(CrossEntropyBackward, k_xent_bwd, "sm100_softmax_xent_backward")
  REG3(NllLoss, k_nll, "sm100_nll_loss") REG3(NllLossBackward, k_nll_bwd, "sm100_nll_loss_backward")
  REG3(Embedding, k_embedding, "sm100_embedding_gather") REG3(EmbeddingBackward, k_embedding_bwd, "sm100_embedding_scatter_add")
  REG3(LayerNorm, k_layernorm, "sm100_layernorm") REG3(LayerNormBackward, k_layernorm_bwd, "sm100_layernorm_backward")
  REG3(CausalSoftmax, k_attn_softmax, "sm100_attention_softmax")
  REG3(CausalSoftmaxBackward, k_attn_softmax_bwd, "sm100_attention_softmax_backward")
  REG3(MaxPool2d, k_maxpool, "sm100_maxpool2d") REG3(MaxPool2dBackward, k_maxpool_bwd, "sm100_maxpool2d_backward")
#undef REG3
}

}  // namespace cu
}  // namespace ob

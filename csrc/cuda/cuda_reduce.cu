// sm_100a reductions: sum / mean (full or along one dim), max with int64 indices and its
// scatter backward, and unbroadcast (gradient reduction to a broadcast source).
//
// Every reduction is deterministic: rows are reduced by warp shuffles and a fixed-order
// shared-memory stage; long reductions are split over blocks into float partials held in
// a scratch lease and summed in a fixed order by a second kernel (no atomics).
//
// Replaces (reference project paths): src/backends/cuda/reduce_kernels.cu:34-800 and the
// atomicAdd-based unbroadcast in src/backends/cuda/binary_kernels.cu:396-590.
#include "ob/cuda_common.cuh"
#include "ob/ops.h"

namespace ob {
namespace cu {
namespace {

constexpr int kThreads = 256;

// in: [outer, reduce] rows (inner == 1).  grid = (splits, outer).  Each block reduces one
// chunk of one row; partial[o * splits + s].
template <class T>
__global__ void row_sum_kernel(const T* __restrict__ in, float* __restrict__ partial, T* __restrict__ out,
                               int64_t reduce, int64_t chunk, int splits, float scale) {
  __shared__ float smem[32];
  const int64_t o = blockIdx.y;
  const int s = blockIdx.x;
  const int64_t begin = static_cast<int64_t>(s) * chunk;
  int64_t end = begin + chunk;
  if (end > reduce) end = reduce;
  const T* row = in + o * reduce;
  float acc = 0.f;
  constexpr int N = Pack<T>::N;
  // Vector body when this chunk starts on a 16-byte boundary.
  int64_t i = begin;
  if ((reinterpret_cast<uintptr_t>(row + begin) & 15u) == 0) {
    const int64_t nv = (end - begin) / N;
    // Four independent 16-byte loads per thread and step keep enough bytes in flight to cover
    // the DRAM latency; the four partial sums are combined in a fixed order.
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
    int64_t v = threadIdx.x;
    for (; v + 3 * static_cast<int64_t>(blockDim.x) < nv; v += 4 * static_cast<int64_t>(blockDim.x)) {
      Pack<T> p[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) p[u] = load_pack(row + begin + (v + u * static_cast<int64_t>(blockDim.x)) * N);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int k = 0; k < N; ++k) a4[u] += to_f(p[u].v[k]);
    }
    for (; v < nv; v += blockDim.x) {
      Pack<T> p = load_pack(row + begin + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) a4[0] += to_f(p.v[k]);
    }
    acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    i = begin + nv * N;
  }
  for (int64_t j = i + threadIdx.x; j < end; j += blockDim.x) acc += to_f(row[j]);
  const float total = block_sum(acc, smem);
  if (threadIdx.x == 0) {
    if (splits == 1) out[o] = from_f<T>(total * scale);
    else partial[o * splits + s] = total;
  }
}

// Short rows (inner == 1, a few thousand elements): one warp per row, shuffles only.
template <class T>
__global__ void row_sum_warp_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t reduce, float scale) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t o = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (o >= rows) return;
  const T* row = in + o * reduce;
  float acc = 0.f;
  int64_t i = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    const int64_t nv = reduce / N;
    for (int64_t v = lane; v < nv; v += 32) {
      const Pack<T> p = load_pack(row + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) acc += to_f(p.v[k]);
    }
    i = nv * N;
  }
  for (int64_t j = i + lane; j < reduce; j += 32) acc += to_f(row[j]);
  acc = warp_sum(acc);
  if (lane == 0) out[o] = from_f<T>(acc * scale);
}

// in: [outer, reduce, inner] with inner > 1.  block = (32, 8); grid = (ceil(inner/32), splits, outer).
template <class T>
__global__ void col_sum_kernel(const T* __restrict__ in, float* __restrict__ partial, T* __restrict__ out,
                               int64_t reduce, int64_t inner, int64_t chunk, int splits, float scale) {
  __shared__ float tile[8][33];
  const int64_t o = blockIdx.z;
  const int s = blockIdx.y;
  const int64_t k = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  const int64_t begin = static_cast<int64_t>(s) * chunk;
  int64_t end = begin + chunk;
  if (end > reduce) end = reduce;
  float acc = 0.f;
  if (k < inner) {
    const T* base = in + o * reduce * inner + k;
    for (int64_t r = begin + threadIdx.y; r < end; r += 8) acc += to_f(base[r * inner]);
  }
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && k < inner) {
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) total += tile[j][threadIdx.x];
    if (splits == 1) out[o * inner + k] = from_f<T>(total * scale);
    else partial[(o * splits + s) * inner + k] = total;
  }
}

// Same reduction with 16-byte loads: every thread owns Pack<T>::N adjacent columns, a warp covers
// 32 * N columns of one row (full 128-byte lines), 8 rows per block step, 4 steps in flight.
// Requires inner % N == 0 and a 16-byte aligned input.
template <class T>
__global__ void col_sum_vec_kernel(const T* __restrict__ in, float* __restrict__ partial, T* __restrict__ out,
                                   int64_t reduce, int64_t inner, int64_t chunk, int splits, float scale) {
  constexpr int N = Pack<T>::N;
  __shared__ float tile[8][32][N + 1];
  const int64_t o = blockIdx.z;
  const int s = blockIdx.y;
  const int64_t k0 = (static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x) * N;
  const int64_t begin = static_cast<int64_t>(s) * chunk;
  int64_t end = begin + chunk;
  if (end > reduce) end = reduce;
  float acc[N];
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = 0.f;
  if (k0 < inner) {
    const T* base = in + o * reduce * inner + k0;
    int64_t r = begin + threadIdx.y;
    for (; r + 24 < end; r += 32) {
      Pack<T> p0 = load_pack(base + r * inner), p1 = load_pack(base + (r + 8) * inner), p2 = load_pack(base + (r + 16) * inner),
              p3 = load_pack(base + (r + 24) * inner);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] += (to_f(p0.v[j]) + to_f(p1.v[j])) + (to_f(p2.v[j]) + to_f(p3.v[j]));
    }
    for (; r < end; r += 8) {
      Pack<T> p0 = load_pack(base + r * inner);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] += to_f(p0.v[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) tile[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && k0 < inner) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float total = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) total += tile[y][threadIdx.x][j];
      if (splits == 1) out[o * inner + k0 + j] = from_f<T>(total * scale);
      else partial[(o * splits + s) * inner + k0 + j] = total;
    }
  }
}

// Second pass of the row sums: out[o] = scale * sum_s partial[o * splits + s].  One warp per
// row: lane l adds partials l, l + 32, ... in order, then a shuffle tree combines the lanes, so
// the result does not depend on scheduling.
template <class T>
__global__ void finalize_rows_kernel(const float* __restrict__ partial, T* __restrict__ out, int64_t outer, int splits, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t o = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (o >= outer) return;
  float total = 0.f;
  for (int s = lane; s < splits; s += 32) total += partial[o * splits + s];
  total = warp_sum(total);
  if (lane == 0) out[o] = from_f<T>(total * scale);
}

// Second pass: out[o, k] = scale * sum_s partial[o, s, k].  Block (32, 8): 32 adjacent outputs,
// eight groups striding over the splits (enough loads in flight for a few hundred KB), then a
// fixed-order sum of the eight partials.  grid = (ceil(inner / 32), outer).
template <class T>
__global__ void finalize_sum_kernel(const float* __restrict__ partial, T* __restrict__ out, int64_t outer,
                                    int64_t inner, int splits, float scale) {
  __shared__ float tile[8][33];
  const int64_t o = blockIdx.y;
  const int64_t k = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  float acc = 0.f;
  if (k < inner) {
    const float* base = partial + o * splits * inner + k;
#pragma unroll 4
    for (int s = threadIdx.y; s < splits; s += 8) acc += base[static_cast<int64_t>(s) * inner];
  }
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && k < inner) {
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) total += tile[j][threadIdx.x];
    out[o * inner + k] = from_f<T>(total * scale);
  }
}

template <class T>
void sum_launch(const T* in, T* out, int64_t outer, int64_t reduce, int64_t inner, float scale, const Tensor& ref,
                cudaStream_t st) {
  const int sms = sm_count_for(ref);
  if (inner == 1) {
    // Aim for ~4 CTAs per SM overall; each split handles at least 4096 elements.
    int64_t want = (static_cast<int64_t>(sms) * 4 + outer - 1) / outer;
    int64_t max_splits = (reduce + 4095) / 4096;
    int splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min(want, max_splits), 1024)));
    int64_t chunk = (reduce + splits - 1) / splits;
    chunk = (chunk + 7) & ~int64_t(7);  // keep chunk starts 16-byte aligned for 2-byte types
    splits = static_cast<int>((reduce + chunk - 1) / chunk);
    if (splits == 1 && reduce <= 8192 && outer >= static_cast<int64_t>(sms) * 8) {
      row_sum_warp_kernel<T><<<static_cast<unsigned>((outer * 32 + kThreads - 1) / kThreads), kThreads, 0, st>>>(in, out, outer, reduce, scale);
      check_launch("row sum");
      return;
    }
    if (outer > 65535) {  // grid.y limit: fall back to one row per block in x
      for (int64_t o0 = 0; o0 < outer; o0 += 65535) {
        const int64_t no = std::min<int64_t>(65535, outer - o0);
        row_sum_kernel<T><<<dim3(1, static_cast<unsigned>(no)), kThreads, 0, st>>>(in + o0 * reduce, nullptr, out + o0,
                                                                               reduce, reduce, 1, scale);
      }
      check_launch("row sum");
      return;
    }
    if (splits == 1) {
      row_sum_kernel<T><<<dim3(1, static_cast<unsigned>(outer)), kThreads, 0, st>>>(in, nullptr, out, reduce, reduce, 1, scale);
      check_launch("row sum");
      return;
    }
    ScratchLease lease(ref.device(), sizeof(float) * outer * splits, st);
    float* partial = static_cast<float*>(lease.data());
    row_sum_kernel<T><<<dim3(splits, static_cast<unsigned>(outer)), kThreads, 0, st>>>(in, partial, out, reduce, chunk, splits, scale);
    finalize_rows_kernel<T><<<static_cast<unsigned>((outer * 32 + kThreads - 1) / kThreads), kThreads, 0, st>>>(partial, out, outer, splits, scale);
    check_launch("row sum (split)");
    return;
  }
  constexpr int VN = Pack<T>::N;
  const bool vec = VN > 1 && inner % VN == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  const int64_t col_blocks = vec ? (inner + 32 * VN - 1) / (32 * VN) : (inner + 31) / 32;
  int64_t want = (static_cast<int64_t>(sms) * 4 + col_blocks * outer - 1) / (col_blocks * outer);
  int64_t max_splits = (reduce + 63) / 64;
  int splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min(want, max_splits), 512)));
  const int64_t chunk = (reduce + splits - 1) / splits;
  splits = static_cast<int>((reduce + chunk - 1) / chunk);
  if (outer > 65535) throw std::invalid_argument("sum: outer extent too large for a strided reduction");
  dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(splits), static_cast<unsigned>(outer));
  if (splits == 1) {
    if (vec) col_sum_vec_kernel<T><<<grid, dim3(32, 8), 0, st>>>(in, nullptr, out, reduce, inner, chunk, 1, scale);
    else col_sum_kernel<T><<<grid, dim3(32, 8), 0, st>>>(in, nullptr, out, reduce, inner, chunk, 1, scale);
    check_launch("column sum");
    return;
  }
  ScratchLease lease(ref.device(), sizeof(float) * outer * splits * inner, st);
  float* partial = static_cast<float*>(lease.data());
  if (vec) col_sum_vec_kernel<T><<<grid, dim3(32, 8), 0, st>>>(in, partial, out, reduce, inner, chunk, splits, scale);
  else col_sum_kernel<T><<<grid, dim3(32, 8), 0, st>>>(in, partial, out, reduce, inner, chunk, splits, scale);
  finalize_sum_kernel<T><<<dim3(static_cast<unsigned>((inner + 31) / 32), static_cast<unsigned>(outer)), dim3(32, 8), 0, st>>>(partial, out, outer, inner, splits, scale);
  check_launch("column sum (split)");
}

template <class T>
void k_sum(OpCall& c) {
  sum_launch<T>(c.in[0].data_as<T>(), c.out[0].data_as<T>(), c.i[0], c.i[1], c.i[2], 1.f, c.in[0], stream_of(c));
}
template <class T>
void k_mean(OpCall& c) {
  sum_launch<T>(c.in[0].data_as<T>(), c.out[0].data_as<T>(), c.i[0], c.i[1], c.i[2],
                static_cast<float>(1.0 / static_cast<double>(c.i[1])), c.in[0], stream_of(c));
}

// ------------------------------------------------------------------------ max
__device__ __forceinline__ bool better(float cv, int64_t ci, float bv, int64_t bi) {
  // First NaN beats numbers; among equals the smaller index wins.
  const bool cn = cv != cv, bn = bv != bv;
  if (cn || bn) {
    if (cn && bn) return ci < bi;
    return cn;
  }
  if (cv > bv) return true;
  if (cv < bv) return false;
  return ci < bi;
}

// One block per (outer, inner) output; threads stride over the reduced extent.
template <class T>
__global__ void max_kernel(const T* __restrict__ in, T* __restrict__ values, int64_t* __restrict__ indices,
                           int64_t reduce, int64_t inner) {
  __shared__ float sv[kThreads];
  __shared__ int64_t si[kThreads];
  const int64_t out_idx = blockIdx.x;
  const int64_t o = out_idx / inner, k = out_idx - o * inner;
  const T* base = in + o * reduce * inner + k;
  float bv = 0.f;
  int64_t bi = -1;
  for (int64_t r = threadIdx.x; r < reduce; r += blockDim.x) {
    const float v = to_f(base[r * inner]);
    if (bi < 0 || better(v, r, bv, bi)) { bv = v; bi = r; }
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int w = blockDim.x / 2; w > 0; w >>= 1) {
    if (threadIdx.x < w) {
      const int64_t oi = si[threadIdx.x + w];
      if (oi >= 0 && (si[threadIdx.x] < 0 || better(sv[threadIdx.x + w], oi, sv[threadIdx.x], si[threadIdx.x]))) {
        sv[threadIdx.x] = sv[threadIdx.x + w];
        si[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    values[out_idx] = base[si[0] * inner];
    indices[out_idx] = si[0];
  }
}

// Row-wise extrema (inner == 1): one warp per row, 16-byte loads, (value, index) pairs merged with
// shuffles under the same policy (first NaN wins, ties go to the smaller index).
template <class T>
__global__ void max_row_warp_kernel(const T* __restrict__ in, T* __restrict__ values, int64_t* __restrict__ indices,
                                    int64_t rows, int64_t reduce) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const T* base = in + row * reduce;
  float bv = 0.f;
  int64_t bi = -1;
  const bool vec = (reduce % N == 0) && ((reinterpret_cast<uintptr_t>(base) & 15u) == 0);
  if (vec) {
    for (int64_t p = lane; p < reduce / N; p += 32) {
      const Pack<T> pk = load_pack(base + p * N);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const float v = to_f(pk.v[k]);
        const int64_t r = p * N + k;
        if (bi < 0 || better(v, r, bv, bi)) { bv = v; bi = r; }
      }
    }
  } else {
    for (int64_t r = lane; r < reduce; r += 32) {
      const float v = to_f(base[r]);
      if (bi < 0 || better(v, r, bv, bi)) { bv = v; bi = r; }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
  }
  if (lane == 0) {
    values[row] = base[bi];
    indices[row] = bi;
  }
}

template <class T>
__global__ void max_scatter_kernel(const T* __restrict__ g, const int64_t* __restrict__ idx, T* __restrict__ out,
                                   int64_t n_out, int64_t reduce, int64_t inner) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_out; i += stride) {
    const int64_t o = i / inner, k = i - o * inner;
    out[(o * reduce + idx[i]) * inner + k] = g[i];
  }
}

template <class T>
void k_max(OpCall& c) {
  const int64_t outer = c.i[0], reduce = c.i[1], inner = c.i[2];
  const int64_t n_out = outer * inner;
  if (n_out > 2147483647LL) throw std::invalid_argument("max: too many outputs");
  if (inner == 1 && reduce >= 64) {
    const int64_t threads_total = n_out * 32;
    max_row_warp_kernel<T><<<static_cast<unsigned>((threads_total + kThreads - 1) / kThreads), kThreads, 0, stream_of(c)>>>(
        c.in[0].data_as<T>(), c.out[0].data_as<T>(), c.out[1].data_as<int64_t>(), n_out, reduce);
    check_launch("max");
    return;
  }
  max_kernel<T><<<static_cast<unsigned>(n_out), kThreads, 0, stream_of(c)>>>(c.in[0].data_as<T>(), c.out[0].data_as<T>(),
                                                                           c.out[1].data_as<int64_t>(), reduce, inner);
  check_launch("max");
}

template <class T>
void k_max_backward(OpCall& c) {
  const int64_t outer = c.i[0], reduce = c.i[1], inner = c.i[2];
  Tensor& out = c.out[0];
  OB_CUDA(cudaMemsetAsync(out.data(), 0, out.nbytes(), stream_of(c)));
  const int64_t n_out = outer * inner;
  max_scatter_kernel<T><<<ew_grid(n_out, kThreads, sm_count_for(out)), kThreads, 0, stream_of(c)>>>(
      c.in[0].data_as<T>(), c.in[1].data_as<int64_t>(), out.data_as<T>(), n_out, reduce, inner);
  check_launch("max_backward");
}

// Unbroadcast = a chain of single-run reductions over each maximal run of broadcast dims.
template <class T>
void k_unbroadcast(OpCall& c) {
  const Tensor& g = c.in[0];
  Tensor& out = c.out[0];
  const Shape& padded = c.list;
  Shape cur = g.shape();
  Tensor src = g;
  cudaStream_t st = stream_of(c);
  const int nd = static_cast<int>(cur.size());
  // Collect runs [b, e) of dims where padded == 1 and cur != 1, processed from the last run
  // to the first so earlier extents stay valid.
  std::vector<std::pair<int, int>> runs;
  for (int d = 0; d < nd;) {
    if (padded[d] == 1 && cur[d] != 1) {
      int e = d;
      while (e < nd && padded[e] == 1) ++e;
      runs.emplace_back(d, e);
      d = e;
    } else {
      ++d;
    }
  }
  if (runs.empty()) {
    OB_CUDA(cudaMemcpyAsync(out.data(), g.data(), out.nbytes(), cudaMemcpyDeviceToDevice, st));
    return;
  }
  for (size_t ri = runs.size(); ri-- > 0;) {
    const auto [b, e] = runs[ri];
    int64_t outer = 1, reduce = 1, inner = 1;
    for (int d = 0; d < b; ++d) outer *= cur[d];
    for (int d = b; d < e; ++d) reduce *= cur[d];
    for (int d = e; d < nd; ++d) inner *= cur[d];
    for (int d = b; d < e; ++d) cur[d] = 1;
    Tensor dst = (ri == 0) ? out : Tensor::empty({outer * inner}, g.dtype(), g.device());
    sum_launch<T>(src.data_as<T>(), dst.data_as<T>(), outer, reduce, inner, 1.f, g, st);
    src = dst;
  }
}

}  // namespace

// Shared with other translation units (bias gradients, loss means).
void sum_rows_f32(const float* in, float* out, int64_t outer, int64_t reduce, int64_t inner, float scale,
                  const Tensor& ref, cudaStream_t st) {
  sum_launch<float>(in, out, outer, reduce, inner, scale, ref, st);
}

void register_cuda_reduce(KernelRegistry& r) {
  const uint8_t packed = kContiguous | kEmpty;
#define REG3(OP, FN, NAME)                                                                                      \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, kMaskF32, packed, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::F16), packed, Capability::None}, FN<__half>, NAME "_f16"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::BF16), packed, Capability::Bf16}, FN<__nv_bfloat16>, NAME "_bf16");
  REG3(Sum, k_sum, "sm100_sum") REG3(Mean, k_mean, "sm100_mean") REG3(Max, k_max, "sm100_max")
  REG3(MaxBackward, k_max_backward, "sm100_max_backward") REG3(Unbroadcast, k_unbroadcast, "sm100_unbroadcast")
#undef REG3
}

}  // namespace cu
}  // namespace ob

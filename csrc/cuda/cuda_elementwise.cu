// sm_100a elementwise family: arithmetic, activations and their backward forms, casts,
// strided copies, fills, dropout masks, finite checks, AMP helpers and the fused
// FP32-master Adam/SGD updates.  All kernels are bandwidth-bound, so contiguous work
// moves 16 bytes per access and grids are sized from the SM count; strided or broadcast
// operands take a generic index-unpacking path (up to 8 dims).
//
// Replaces (reference project paths): src/backends/cuda/{binary_kernels,unary_kernels,
// cast_kernels}.cu and the transfer helpers in src/backends/cuda/adapters.cpp.
#include <cstdlib>
#include <atomic>
#include <type_traits>
#include <vector>

#include "ob/cuda_common.cuh"

namespace ob {
namespace cu {

int sm_count_for(const Tensor& t) { return Runtime::instance().cuda(t.device().index).sm_count(); }

static std::atomic<uint64_t> g_launches{0};
uint64_t kernel_launch_count() { return g_launches.load(); }

unsigned int take_index_errors();

// Called once per kernel wrapper after its launches; also counts the wrapper for the
// launch statistics the benchmarks report.
//
// ORTHON_DEBUG_BOUNDS=1 turns every wrapper into a checkpoint: the device is drained, an
// asynchronous fault is reported against the wrapper that caused it, and an index that a kernel
// had to clamp (embedding ids, class targets) raises std::out_of_range naming the wrapper, instead
// of only being counted.
void check_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA launch failed in ") + what + ": " + cudaGetErrorString(e));
  static const bool debug_bounds = [] {
    const char* v = std::getenv("ORTHON_DEBUG_BOUNDS");
    return v != nullptr && v[0] == '1';
  }();
  if (!debug_bounds) return;
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA kernel failed in ") + what + ": " + cudaGetErrorString(e));
  const unsigned int clamped = take_index_errors();
  if (clamped != 0)
    throw std::out_of_range(std::string(what) + ": " + std::to_string(clamped) + " index value(s) outside the valid range");
}

namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------- functors
struct FAdd { __device__ float operator()(float a, float b) const { return a + b; } };
struct FMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct FAddS { float s; __device__ float operator()(float a) const { return a + s; } };
struct FMulS { float s; __device__ float operator()(float a) const { return a * s; } };
struct FNeg { __device__ float operator()(float a) const { return -a; } };
struct FRelu { __device__ float operator()(float a) const { return a > 0.f ? a : 0.f; } };
struct FSigmoid { __device__ float operator()(float a) const { return 1.f / (1.f + __expf(-a)); } };
struct FTanh { __device__ float operator()(float a) const { return tanhf(a); } };
struct FLeaky { float s; __device__ float operator()(float a) const { return a > 0.f ? a : s * a; } };
struct FGelu { __device__ float operator()(float a) const { return 0.5f * a * (1.f + erff(a * 0.70710678118654752f)); } };
struct FExp { __device__ float operator()(float a) const { return expf(a); } };
struct FSqrt { __device__ float operator()(float a) const { return sqrtf(a); } };
struct FRecip { __device__ float operator()(float a) const { return 1.f / a; } };
struct FLog { __device__ float operator()(float a) const { return logf(a); } };
// backward forms: (x, g) -> dx
struct BRelu { __device__ float operator()(float x, float g) const { return x > 0.f ? g : 0.f; } };
struct BSigmoid { __device__ float operator()(float x, float g) const { const float s = 1.f / (1.f + __expf(-x)); return g * s * (1.f - s); } };
struct BTanh { __device__ float operator()(float x, float g) const { const float t = tanhf(x); return g * (1.f - t * t); } };
struct BLeaky { float s; __device__ float operator()(float x, float g) const { return x > 0.f ? g : s * g; } };
struct BGelu {
  __device__ float operator()(float x, float g) const {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return g * (cdf + x * pdf);
  }
};
struct BExp { __device__ float operator()(float x, float g) const { return g * expf(x); } };
struct BSqrt { __device__ float operator()(float x, float g) const { return g / (2.f * sqrtf(x)); } };
struct BRecip { __device__ float operator()(float x, float g) const { return -g / (x * x); } };

// ------------------------------------------------------------ generic kernels
template <class T, class Op>
__global__ void map1_vec(const T* __restrict__ a, T* __restrict__ o, int64_t n, Op op) {
  constexpr int N = Pack<T>::N;
  const int64_t nv = n / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Pack<T> pa = load_pack(a + i * N), po;
#pragma unroll
    for (int k = 0; k < N; ++k) po.v[k] = from_f<T>(op(to_f(pa.v[k])));
    store_pack(o + i * N, po);
  }
  for (int64_t i = nv * N + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    o[i] = from_f<T>(op(to_f(a[i])));
}

template <class T, class Op>
__global__ void map2_vec(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ o, int64_t n, Op op) {
  constexpr int N = Pack<T>::N;
  const int64_t nv = n / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Pack<T> pa = load_pack(a + i * N), pb = load_pack(b + i * N), po;
#pragma unroll
    for (int k = 0; k < N; ++k) po.v[k] = from_f<T>(op(to_f(pa.v[k]), to_f(pb.v[k])));
    store_pack(o + i * N, po);
  }
  for (int64_t i = nv * N + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    o[i] = from_f<T>(op(to_f(a[i]), to_f(b[i])));
}

// One operand has the output's shape, the other is broadcast along leading dimensions (MODE 1:
// a bias row, index = linear % inner) or along trailing ones (MODE 2: one value per row, index =
// linear / inner; a scalar is the case inner == n).  inner and n are multiples of the pack width,
// so a pack never straddles a row.  SWAP: the broadcast operand is the left argument of op.
template <class T, class Op, int MODE, bool SWAP>
__global__ void map2_bcast_vec(const T* __restrict__ full, const T* __restrict__ small, T* __restrict__ o, int64_t n,
                               int64_t inner, Op op) {
  constexpr int N = Pack<T>::N;
  const int64_t nv = n / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const int64_t lin = i * N;
    Pack<T> pf = load_pack(full + lin), ps, po;
    if (MODE == 1) {
      ps = load_pack(small + lin % inner);
    } else {
      const T v = small[lin / inner];
#pragma unroll
      for (int k = 0; k < N; ++k) ps.v[k] = v;
    }
#pragma unroll
    for (int k = 0; k < N; ++k)
      po.v[k] = from_f<T>(SWAP ? op(to_f(ps.v[k]), to_f(pf.v[k])) : op(to_f(pf.v[k]), to_f(ps.v[k])));
    store_pack(o + lin, po);
  }
}

__device__ __forceinline__ void unpack(const Strided& s, int64_t lin, int64_t& o0, int64_t& o1, int64_t& o2) {
  o0 = o1 = o2 = 0;
#pragma unroll 1
  for (int d = s.nd - 1; d >= 0; --d) {
    const int64_t q = lin / s.shape[d];
    const int64_t r = lin - q * s.shape[d];
    o0 += r * s.st[0][d];
    o1 += r * s.st[1][d];
    o2 += r * s.st[2][d];
    lin = q;
  }
}

template <class T, class Op>
__global__ void map1_strided(const T* __restrict__ a, T* __restrict__ o, int64_t n, Strided s, Op op) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo, oa, ob_;
    unpack(s, i, oo, oa, ob_);
    o[oo] = from_f<T>(op(to_f(a[oa])));
  }
}

template <class T, class Op>
__global__ void map2_strided(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ o, int64_t n,
                             Strided s, Op op) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo, oa, ob_;
    unpack(s, i, oo, oa, ob_);
    o[oo] = from_f<T>(op(to_f(a[oa]), to_f(b[ob_])));
  }
}

// Byte-wise strided copy for any element size (1, 2, 4 or 8 bytes).
template <class U>
__global__ void copy_strided(const U* __restrict__ a, U* __restrict__ o, int64_t n, Strided s) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo, oa, ob_;
    unpack(s, i, oo, oa, ob_);
    o[oo] = a[oa];
  }
}

// 2-D transpose-like copies go through a 32x33 shared tile so both sides coalesce.
template <class U>
__global__ void transpose_tiled(const U* __restrict__ a, U* __restrict__ o, int64_t rows, int64_t cols,
                                int64_t a_rs, int64_t a_cs, int64_t batch_a, int64_t batch_o) {
  // out[r, c] (contiguous, cols fastest) = a[r*a_rs + c*a_cs] where a_rs == 1 (source is column-major)
  __shared__ U tile[32][33];
  const int64_t b = blockIdx.z;
  const U* ab = a + b * batch_a;
  U* ob_ = o + b * batch_o;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32, r0 = static_cast<int64_t>(blockIdx.y) * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (c < cols && r < rows) tile[j][threadIdx.x] = ab[r * a_rs + c * a_cs];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) ob_[r * cols + c] = tile[threadIdx.x][j];
  }
}

template <class T> struct is_lowp { static constexpr bool value = false; };
template <> struct is_lowp<__half> { static constexpr bool value = true; };
template <> struct is_lowp<__nv_bfloat16> { static constexpr bool value = true; };

template <class S, class D>
__device__ __forceinline__ D conv(S v) {
  if constexpr (is_lowp<S>::value && is_lowp<D>::value) {
    return from_f<D>(to_f(v));
  } else if constexpr (is_lowp<S>::value) {
    const float f = to_f(v);
    if constexpr (std::is_same<D, bool>::value) return f != 0.f;
    else return static_cast<D>(f);
  } else if constexpr (is_lowp<D>::value) {
    return from_f<D>(static_cast<float>(v));
  } else if constexpr (std::is_same<D, bool>::value) {
    return v != S(0);
  } else {
    return static_cast<D>(v);
  }
}

template <class S, class D>
__global__ void cast_kernel(const S* __restrict__ a, D* __restrict__ o, int64_t n, Strided s, bool packed) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo = i, oa = i, ob_ = 0;
    if (!packed) unpack(s, i, oo, oa, ob_);
    o[oo] = conv<S, D>(a[oa]);
  }
}

template <class U>
__global__ void fill_kernel(U* __restrict__ o, int64_t n, U value, Strided s, bool packed) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo = i, oa, ob_;
    if (!packed) unpack(s, i, oo, oa, ob_);
    o[oo] = value;
  }
}

template <class T>
__global__ void add_inplace_kernel(T* __restrict__ a, const T* __restrict__ b, int64_t n, float alpha) {
  constexpr int N = Pack<T>::N;
  const int64_t nv = n / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Pack<T> pa = load_pack(a + i * N), pb = load_pack(b + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) pa.v[k] = from_f<T>(to_f(pa.v[k]) + alpha * to_f(pb.v[k]));
    store_pack(a + i * N, pa);
  }
  for (int64_t i = nv * N + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    a[i] = from_f<T>(to_f(a[i]) + alpha * to_f(b[i]));
}

template <class T>
__global__ void add_inplace_strided(T* __restrict__ a, const T* __restrict__ b, int64_t n, float alpha, Strided s) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oa, ob_, o2;
    unpack(s, i, oa, ob_, o2);
    a[oa] = from_f<T>(to_f(a[oa]) + alpha * to_f(b[ob_]));
  }
}

__device__ __forceinline__ float dropout_value(uint64_t x, float p, float scale) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  x = x ^ (x >> 31);
  const float r = static_cast<float>(static_cast<uint32_t>(x >> 40)) * (1.0f / 16777216.0f);
  return r >= p ? scale : 0.f;
}

// Element i of the mask depends only on seed + i, so each thread produces one 16-byte pack.
template <class T>
__global__ void dropout_mask_kernel(T* __restrict__ o, int64_t n, float p, float scale, uint64_t seed, bool vec) {
  constexpr int N = Pack<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nv = vec ? n / N : 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Pack<T> po;
#pragma unroll
    for (int k = 0; k < N; ++k) po.v[k] = from_f<T>(dropout_value(seed + static_cast<uint64_t>(i * N + k), p, scale));
    store_pack(o + i * N, po);
  }
  for (int64_t i = nv * N + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    o[i] = from_f<T>(dropout_value(seed + static_cast<uint64_t>(i), p, scale));
}

// Fused dropout: o[i] = x[i] * mask(seed + i) in one pass (the mask is never stored; the backward
// pass runs the same kernel on the gradient).
template <class T>
__global__ void dropout_apply_kernel(const T* __restrict__ x, T* __restrict__ o, int64_t n, float p, float scale, uint64_t seed, bool vec) {
  constexpr int N = Pack<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nv = vec ? n / N : 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const Pack<T> px = load_pack(x + i * N);
    Pack<T> po;
#pragma unroll
    for (int k = 0; k < N; ++k) {
      // The product is rounded from the rounded mask value, as the two-kernel form does.
      const float m = to_f(from_f<T>(dropout_value(seed + static_cast<uint64_t>(i * N + k), p, scale)));
      po.v[k] = from_f<T>(to_f(px.v[k]) * m);
    }
    store_pack(o + i * N, po);
  }
  for (int64_t i = nv * N + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    o[i] = from_f<T>(to_f(x[i]) * to_f(from_f<T>(dropout_value(seed + static_cast<uint64_t>(i), p, scale))));
}

template <class T>
__global__ void finite_kernel(const T* __restrict__ a, int64_t n, Strided s, bool packed, int* flag) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool bad = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oo = i, oa, ob_;
    if (!packed) unpack(s, i, oo, oa, ob_);
    const float v = to_f(a[oo]);
    bad |= !isfinite(v);
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 1);
}

template <class T>
__global__ void unscale_kernel(const T* __restrict__ g, float* __restrict__ o, int64_t n, float inv, int* flag) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool bad = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = to_f(g[i]) * inv;
    bad |= !isfinite(v);
    o[i] = v;
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 1);
}

template <class T>
__global__ void amp_copy_kernel(T* __restrict__ model, const float* __restrict__ master, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    model[i] = from_f<T>(master[i]);
}

struct AdamArgs { float lr, b1, b2, eps, wd, inv_bc1, inv_bc2, gs; };

// One pass: read grad (any float dtype), update fp32 master + moments, optionally write
// the low-precision model copy.  Formula order matches the composed optimizer: decoupled
// decay first, epsilon outside the square root.
template <class G, class M>
__global__ void adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                            const G* __restrict__ g, M* __restrict__ model, int64_t n, AdamArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gr = to_f(g[i]) * a.gs;
    float mi = m[i], vi = v[i], w = p[i];
    mi = mi + (a.b1 - 1.f) * mi;
    mi = mi + (1.f - a.b1) * gr;
    vi = vi + (a.b2 - 1.f) * vi;
    vi = vi + (1.f - a.b2) * (gr * gr);
    const float denom = sqrtf(vi * a.inv_bc2) + a.eps;
    if (a.wd != 0.f) w = w + (-a.lr * a.wd) * w;
    w = w + (-a.lr * a.inv_bc1) * (mi / denom);
    m[i] = mi;
    v[i] = vi;
    p[i] = w;
    if (model != nullptr) model[i] = from_f<M>(w);
  }
}

// 16-byte accesses: loads and stores of 8 consecutive elements of any of the element types.
template <class E>
__device__ __forceinline__ void load8(const E* p, float* out) {
  if (sizeof(E) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const E* e = reinterpret_cast<const E*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = to_f(e[k]);
  }
}
template <class E>
__device__ __forceinline__ void store8(E* p, const float* in) {
  if (sizeof(E) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(in[4], in[5], in[6], in[7]);
  } else {
    uint4 raw;
    E* e = reinterpret_cast<E*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) e[k] = from_f<E>(in[k]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
}

// Vector form of adam_kernel over the first n8 * 8 elements (every pointer 16-byte aligned).
template <class G, class M>
__global__ void adam_vec_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                const G* __restrict__ g, M* __restrict__ model, int64_t n8, AdamArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const int64_t e = i * 8;
    float gr[8], mi[8], vi[8], w[8];
    load8(g + e, gr);
    load8(m + e, mi);
    load8(v + e, vi);
    load8(p + e, w);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = gr[k] * a.gs;
      mi[k] = mi[k] + (a.b1 - 1.f) * mi[k];
      mi[k] = mi[k] + (1.f - a.b1) * gk;
      vi[k] = vi[k] + (a.b2 - 1.f) * vi[k];
      vi[k] = vi[k] + (1.f - a.b2) * (gk * gk);
      const float denom = sqrtf(vi[k] * a.inv_bc2) + a.eps;
      if (a.wd != 0.f) w[k] = w[k] + (-a.lr * a.wd) * w[k];
      w[k] = w[k] + (-a.lr * a.inv_bc1) * (mi[k] / denom);
    }
    store8(m + e, mi);
    store8(v + e, vi);
    store8(p + e, w);
    if (model != nullptr) store8(model + e, w);
  }
}

template <class G, class M>
__global__ void sgd_vec_kernel(float* __restrict__ p, const G* __restrict__ g, M* __restrict__ model, int64_t n8,
                               float lr, float wd, float gs) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const int64_t e = i * 8;
    float gr[8], w[8];
    load8(g + e, gr);
    load8(p + e, w);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (wd != 0.f) w[k] = w[k] + (-lr * wd) * w[k];
      w[k] = w[k] + (-lr) * (gr[k] * gs);
    }
    store8(p + e, w);
    if (model != nullptr) store8(model + e, w);
  }
}

inline bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr, const void* e = nullptr) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
           reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(e)) & 15u) == 0;
}

template <class G, class M>
__global__ void sgd_kernel(float* __restrict__ p, const G* __restrict__ g, M* __restrict__ model, int64_t n,
                           float lr, float wd, float gs) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float w = p[i];
    if (wd != 0.f) w = w + (-lr * wd) * w;
    w = w + (-lr) * (to_f(g[i]) * gs);
    p[i] = w;
    if (model != nullptr) model[i] = from_f<M>(w);
  }
}

// --------------------------------------------------------------- host helpers
Strided make_strided(const Shape& shape, const Shape* s0, const Shape* s1, const Shape* s2) {
  Strided s{};
  if (shape.size() > 8) throw std::invalid_argument("tensors with more than 8 dimensions are not supported on CUDA");
  s.nd = static_cast<int>(shape.size());
  for (int d = 0; d < s.nd; ++d) {
    s.shape[d] = shape[d];
    s.st[0][d] = s0 ? (*s0)[d] : 0;
    s.st[1][d] = s1 ? (*s1)[d] : 0;
    s.st[2][d] = s2 ? (*s2)[d] : 0;
  }
  return s;
}

Shape bstrides(const Tensor& t, const Shape& out_shape) {
  const int nd = static_cast<int>(out_shape.size()), td = t.ndim();
  Shape st(nd, 0);
  for (int i = 0; i < td; ++i) {
    const int o = nd - td + i;
    st[o] = (t.shape()[i] == 1 && out_shape[o] != 1) ? 0 : t.strides()[i];
  }
  return st;
}

template <class T, class Op>
void launch_map1(OpCall& c, Op op) {
  const Tensor& a = c.in[0];
  Tensor& o = c.out[0];
  const int64_t n = o.numel();
  const int sms = sm_count_for(o);
  if (a.is_contiguous() && aligned16(a.data()) && aligned16(o.data())) {
    map1_vec<T, Op><<<ew_grid(n / Pack<T>::N + 1, kThreads, sms), kThreads, 0, stream_of(c)>>>(
        a.data_as<T>(), o.data_as<T>(), n, op);
  } else {
    const Strided s = make_strided(o.shape(), &o.strides(), &a.strides(), nullptr);
    map1_strided<T, Op><<<ew_grid(n, kThreads, sms), kThreads, 0, stream_of(c)>>>(a.data_as<T>(), o.data_as<T>(), n, s, op);
  }
  check_launch("elementwise map");
}

// Fast path for `full (op) small` where `small` is a contiguous row (trailing dimensions of the
// output), a contiguous column (leading dimensions, then ones) or a single value.  Returns false
// when the operands do not have that form.
template <class T, class Op>
bool launch_map2_bcast(const Tensor& full, const Tensor& small, Tensor& o, cudaStream_t st, Op op, bool swap) {
  constexpr int N = Pack<T>::N;
  const int64_t n = o.numel();
  if (n == 0 || n % N != 0 || full.shape() != o.shape() || !full.is_contiguous() || !small.is_contiguous() || !o.is_contiguous() ||
      small.numel() >= n || small.numel() == 0 || !aligned16(full.data()) || !aligned16(o.data()))
    return false;
  const int nd = o.ndim(), sd = small.ndim();
  if (sd > nd) return false;
  Shape padded(nd, 1);
  for (int i = 0; i < sd; ++i) padded[nd - sd + i] = small.shape()[i];
  // Split point d: row form = ones before d, output sizes from d on; column form = output sizes
  // before d, ones from d on.
  int mode = 0;
  int64_t inner = 1;
  for (int d = 0; d <= nd && !mode; ++d) {
    bool row = true, col = true;
    for (int k = 0; k < nd; ++k) {
      const int64_t want_row = k < d ? 1 : o.shape()[k], want_col = k < d ? o.shape()[k] : 1;
      row = row && padded[k] == want_row;
      col = col && padded[k] == want_col;
    }
    if (row || col) {
      inner = 1;
      for (int k = d; k < nd; ++k) inner *= o.shape()[k];
      mode = row ? 1 : 2;
    }
  }
  if (!mode || inner % N != 0) return false;
  if (mode == 1 && !aligned16(small.data())) return false;
  const int sms = sm_count_for(o);
  const int grid = ew_grid(n / N, kThreads, sms);
  const T* f = full.data_as<T>();
  const T* sm = small.data_as<T>();
  T* out = o.data_as<T>();
  if (mode == 1) {
    if (swap) map2_bcast_vec<T, Op, 1, true><<<grid, kThreads, 0, st>>>(f, sm, out, n, inner, op);
    else map2_bcast_vec<T, Op, 1, false><<<grid, kThreads, 0, st>>>(f, sm, out, n, inner, op);
  } else {
    if (swap) map2_bcast_vec<T, Op, 2, true><<<grid, kThreads, 0, st>>>(f, sm, out, n, inner, op);
    else map2_bcast_vec<T, Op, 2, false><<<grid, kThreads, 0, st>>>(f, sm, out, n, inner, op);
  }
  return true;
}

template <class T, class Op>
void launch_map2(const Tensor& a, const Tensor& b, Tensor& o, cudaStream_t st, Op op) {
  const int64_t n = o.numel();
  const int sms = sm_count_for(o);
  if (a.is_contiguous() && b.is_contiguous() && a.shape() == o.shape() && b.shape() == o.shape() &&
      aligned16(a.data()) && aligned16(b.data()) && aligned16(o.data())) {
    map2_vec<T, Op><<<ew_grid(n / Pack<T>::N + 1, kThreads, sms), kThreads, 0, st>>>(a.data_as<T>(), b.data_as<T>(),
                                                                                     o.data_as<T>(), n, op);
  } else if (launch_map2_bcast<T>(a, b, o, st, op, false) || launch_map2_bcast<T>(b, a, o, st, op, true)) {
  } else {
    const Shape sa = bstrides(a, o.shape()), sb = bstrides(b, o.shape());
    const Strided s = make_strided(o.shape(), &o.strides(), &sa, &sb);
    map2_strided<T, Op><<<ew_grid(n, kThreads, sms), kThreads, 0, st>>>(a.data_as<T>(), b.data_as<T>(), o.data_as<T>(), n, s, op);
  }
  check_launch("elementwise binary");
}

template <class T> void k_add(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), FAdd{}); }
template <class T> void k_mul(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), FMul{}); }
template <class T> void k_add_scalar(OpCall& c) { launch_map1<T>(c, FAddS{static_cast<float>(c.f[0])}); }
template <class T> void k_mul_scalar(OpCall& c) { launch_map1<T>(c, FMulS{static_cast<float>(c.f[0])}); }
template <class T> void k_neg(OpCall& c) { launch_map1<T>(c, FNeg{}); }
template <class T> void k_relu(OpCall& c) { launch_map1<T>(c, FRelu{}); }
template <class T> void k_sigmoid(OpCall& c) { launch_map1<T>(c, FSigmoid{}); }
template <class T> void k_tanh(OpCall& c) { launch_map1<T>(c, FTanh{}); }
template <class T> void k_leaky(OpCall& c) { launch_map1<T>(c, FLeaky{static_cast<float>(c.f[0])}); }
template <class T> void k_gelu(OpCall& c) { launch_map1<T>(c, FGelu{}); }
template <class T> void k_exp(OpCall& c) { launch_map1<T>(c, FExp{}); }
template <class T> void k_sqrt(OpCall& c) { launch_map1<T>(c, FSqrt{}); }
template <class T> void k_recip(OpCall& c) { launch_map1<T>(c, FRecip{}); }
template <class T> void k_log(OpCall& c) { launch_map1<T>(c, FLog{}); }
template <class T> void k_relu_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BRelu{}); }
template <class T> void k_sigmoid_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BSigmoid{}); }
template <class T> void k_tanh_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BTanh{}); }
template <class T> void k_leaky_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BLeaky{static_cast<float>(c.f[0])}); }
template <class T> void k_gelu_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BGelu{}); }
template <class T> void k_exp_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BExp{}); }
template <class T> void k_sqrt_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BSqrt{}); }
template <class T> void k_recip_b(OpCall& c) { launch_map2<T>(c.in[0], c.in[1], c.out[0], stream_of(c), BRecip{}); }

template <class T>
void k_add_inplace(OpCall& c) {
  Tensor& a = c.in[0];
  const Tensor& b = c.in[1];
  const int64_t n = a.numel();
  const int sms = sm_count_for(a);
  if (a.is_contiguous() && b.is_contiguous() && a.shape() == b.shape() && aligned16(a.data()) && aligned16(b.data())) {
    add_inplace_kernel<T><<<ew_grid(n / Pack<T>::N + 1, kThreads, sms), kThreads, 0, stream_of(c)>>>(
        a.data_as<T>(), b.data_as<T>(), n, static_cast<float>(c.f[0]));
  } else {
    const Shape sb = bstrides(b, a.shape());
    const Strided s = make_strided(a.shape(), &a.strides(), &sb, nullptr);
    add_inplace_strided<T><<<ew_grid(n, kThreads, sms), kThreads, 0, stream_of(c)>>>(a.data_as<T>(), b.data_as<T>(), n,
                                                                                    static_cast<float>(c.f[0]), s);
  }
  check_launch("add_");
}

template <class T>
void k_mul_inplace(OpCall& c) {
  OpCall d;
  d.in[0] = c.in[0];
  d.out[0] = c.in[0];
  d.stream = c.stream;
  launch_map1<T>(d, FMulS{static_cast<float>(c.f[0])});
}

template <class U>
void copy_typed(const Tensor& src, Tensor& dst, cudaStream_t st) {
  const int64_t n = dst.numel();
  const int sms = sm_count_for(dst);
  // Batched 2-D transposes (source column-major in its last two dims) use the tiled path.
  const int nd = dst.ndim();
  if (nd >= 2 && dst.is_contiguous() && src.shape() == dst.shape() && src.strides()[nd - 2] == 1 && nd <= 3 &&
      dst.shape()[nd - 1] > 1 && dst.shape()[nd - 2] > 1) {
    const int64_t rows = dst.shape()[nd - 2], cols = dst.shape()[nd - 1];
    const int64_t nb = nd == 3 ? dst.shape()[0] : 1;
    if (nb <= 65535) {
      dim3 grid(static_cast<unsigned>((cols + 31) / 32), static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>(nb));
      transpose_tiled<U><<<grid, dim3(32, 8), 0, st>>>(static_cast<const U*>(src.data()), static_cast<U*>(dst.data()), rows, cols,
                                                     1, src.strides()[nd - 1], nd == 3 ? src.strides()[0] : 0, rows * cols);
      check_launch("tiled transpose");
      return;
    }
  }
  const Shape ss = bstrides(src, dst.shape());
  const Strided s = make_strided(dst.shape(), &dst.strides(), &ss, nullptr);
  copy_strided<U><<<ew_grid(n, kThreads, sms), kThreads, 0, st>>>(static_cast<const U*>(src.data()), static_cast<U*>(dst.data()), n, s);
  check_launch("strided copy");
}

}  // namespace

void strided_copy_cuda(const Tensor& src, Tensor& dst, cudaStream_t st) {
  if (dst.numel() == 0) return;
  if (src.is_contiguous() && dst.is_contiguous() && src.shape() == dst.shape()) {
    OB_CUDA(cudaMemcpyAsync(dst.data(), src.data(), dst.nbytes(), cudaMemcpyDeviceToDevice, st));
    return;
  }
  switch (dtype_size(dst.dtype())) {
    case 1: copy_typed<uint8_t>(src, dst, st); break;
    case 2: copy_typed<uint16_t>(src, dst, st); break;
    case 4: copy_typed<uint32_t>(src, dst, st); break;
    default: copy_typed<uint64_t>(src, dst, st); break;
  }
}

namespace {

void k_contiguous(OpCall& c) { strided_copy_cuda(c.in[0], c.out[0], stream_of(c)); }

template <class S>
void cast_from(OpCall& c) {
  const Tensor& a = c.in[0];
  Tensor& o = c.out[0];
  const int64_t n = o.numel();
  const bool packed = a.is_contiguous() && o.is_contiguous();
  const Strided s = make_strided(o.shape(), &o.strides(), &a.strides(), nullptr);
  const int grid = ew_grid(n, kThreads, sm_count_for(o));
  cudaStream_t st = stream_of(c);
  const S* pa = a.data_as<S>();
#define CAST_TO(DT, CT) case DType::DT: cast_kernel<S, CT><<<grid, kThreads, 0, st>>>(pa, o.data_as<CT>(), n, s, packed); break;
  switch (o.dtype()) {
    CAST_TO(F32, float) CAST_TO(F64, double) CAST_TO(F16, __half) CAST_TO(BF16, __nv_bfloat16)
    CAST_TO(I32, int32_t) CAST_TO(I64, int64_t) CAST_TO(U8, uint8_t) CAST_TO(I8, int8_t)
    case DType::Bool: cast_kernel<S, bool><<<grid, kThreads, 0, st>>>(pa, o.data_as<bool>(), n, s, packed); break;
    default: throw std::invalid_argument("cast: unsupported target dtype");
  }
#undef CAST_TO
  check_launch("cast");
}

void k_cast(OpCall& c) {
  switch (c.in[0].dtype()) {
    case DType::F32: cast_from<float>(c); break;
    case DType::F64: cast_from<double>(c); break;
    case DType::F16: cast_from<__half>(c); break;
    case DType::BF16: cast_from<__nv_bfloat16>(c); break;
    case DType::I32: cast_from<int32_t>(c); break;
    case DType::I64: cast_from<int64_t>(c); break;
    case DType::U8: cast_from<uint8_t>(c); break;
    case DType::I8: cast_from<int8_t>(c); break;
    case DType::Bool: cast_from<bool>(c); break;
    default: throw std::invalid_argument("cast: unsupported source dtype");
  }
}

void k_fill(OpCall& c) {
  Tensor& t = c.in[0];
  const int64_t n = t.numel();
  const bool packed = t.is_contiguous();
  if (packed && c.f[0] == 0.0) {
    OB_CUDA(cudaMemsetAsync(t.data(), 0, t.nbytes(), stream_of(c)));
    return;
  }
  uint64_t bits = 0;
  store_from_double(&bits, t.dtype(), c.f[0]);
  const Strided s = make_strided(t.shape(), &t.strides(), nullptr, nullptr);
  const int grid = ew_grid(n, kThreads, sm_count_for(t));
  cudaStream_t st = stream_of(c);
  switch (dtype_size(t.dtype())) {
    case 1: fill_kernel<uint8_t><<<grid, kThreads, 0, st>>>(t.data_as<uint8_t>(), n, static_cast<uint8_t>(bits), s, packed); break;
    case 2: fill_kernel<uint16_t><<<grid, kThreads, 0, st>>>(t.data_as<uint16_t>(), n, static_cast<uint16_t>(bits), s, packed); break;
    case 4: fill_kernel<uint32_t><<<grid, kThreads, 0, st>>>(t.data_as<uint32_t>(), n, static_cast<uint32_t>(bits), s, packed); break;
    default: fill_kernel<uint64_t><<<grid, kThreads, 0, st>>>(t.data_as<uint64_t>(), n, bits, s, packed); break;
  }
  check_launch("fill");
}

void k_copy_range(OpCall& c) {
  Tensor& dst = c.in[0];
  const Tensor& src = c.in[1];
  const size_t esz = dtype_size(dst.dtype());
  OB_CUDA(cudaMemcpyAsync(static_cast<char*>(dst.data()) + c.i[0] * esz, static_cast<const char*>(src.data()) + c.i[1] * esz,
                          c.i[2] * esz, cudaMemcpyDeviceToDevice, stream_of(c)));
}

template <class T>
void k_dropout_mask(OpCall& c) {
  Tensor& o = c.out[0];
  const float p = static_cast<float>(c.f[0]);
  if (c.in[0].defined()) {  // fused form: out = in * mask
    const Tensor& x = c.in[0];
    const bool vec2 = aligned16(o.data()) && aligned16(x.data());
    dropout_apply_kernel<T><<<ew_grid(vec2 ? o.numel() / Pack<T>::N + 1 : o.numel(), kThreads, sm_count_for(o)), kThreads, 0, stream_of(c)>>>(
        x.data_as<T>(), o.data_as<T>(), o.numel(), p, 1.0f / (1.0f - p), static_cast<uint64_t>(c.i[0]), vec2);
    check_launch("dropout");
    return;
  }
  const bool vec = aligned16(o.data());
  dropout_mask_kernel<T><<<ew_grid(vec ? o.numel() / Pack<T>::N + 1 : o.numel(), kThreads, sm_count_for(o)), kThreads, 0, stream_of(c)>>>(
      o.data_as<T>(), o.numel(), p, 1.0f / (1.0f - p), static_cast<uint64_t>(c.i[0]), vec);
  check_launch("dropout_mask");
}

// Device flag protocol shared by the two checks below: one int zeroed on the stream,
// set by any block that sees a non-finite value, read back after a stream sync.
int read_flag(Tensor& flag, cudaStream_t st) {
  int host = 0;
  OB_CUDA(cudaMemcpyAsync(&host, flag.data(), sizeof(int), cudaMemcpyDeviceToHost, st));
  OB_CUDA(cudaStreamSynchronize(st));
  return host;
}

void k_isfinite(OpCall& c) {
  const Tensor& t = c.in[0];
  c.i[0] = 1;
  if (!dtype_is_floating(t.dtype())) return;
  const bool shared_flag = c.in[1].defined();  // caller accumulates over many tensors and reads once
  Tensor flag = shared_flag ? c.in[1] : Tensor::zeros({1}, DType::I32, t.device());
  const int64_t n = t.numel();
  const bool packed = t.is_contiguous();
  const Strided s = make_strided(t.shape(), &t.strides(), nullptr, nullptr);
  const int grid = ew_grid(n, kThreads, sm_count_for(t));
  cudaStream_t st = stream_of(c);
  int* pf = flag.data_as<int>();
  switch (t.dtype()) {
    case DType::F32: finite_kernel<float><<<grid, kThreads, 0, st>>>(t.data_as<float>(), n, s, packed, pf); break;
    case DType::F64: finite_kernel<double><<<grid, kThreads, 0, st>>>(t.data_as<double>(), n, s, packed, pf); break;
    case DType::F16: finite_kernel<__half><<<grid, kThreads, 0, st>>>(t.data_as<__half>(), n, s, packed, pf); break;
    default: finite_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(t.data_as<__nv_bfloat16>(), n, s, packed, pf); break;
  }
  check_launch("isfinite_all");
  c.i[0] = shared_flag ? 1 : (read_flag(flag, st) ? 0 : 1);
}

void k_amp_unscale(OpCall& c) {
  Tensor g = c.in[0];
  if (!g.is_contiguous()) {
    Tensor packed = Tensor::empty(g.shape(), g.dtype(), g.device());
    strided_copy_cuda(g, packed, stream_of(c));
    g = packed;
  }
  Tensor& o = c.out[0];
  // A caller-provided flag (in1) accumulates over many tensors and is read by the caller
  // once; without it the result is read back here.
  const bool shared_flag = c.in[1].defined();
  Tensor flag = shared_flag ? c.in[1] : Tensor::zeros({1}, DType::I32, g.device());
  const int64_t n = g.numel();
  const int grid = ew_grid(n, kThreads, sm_count_for(g));
  cudaStream_t st = stream_of(c);
  const float inv = static_cast<float>(c.f[0]);
  int* pf = flag.data_as<int>();
  switch (g.dtype()) {
    case DType::F32: unscale_kernel<float><<<grid, kThreads, 0, st>>>(g.data_as<float>(), o.data_as<float>(), n, inv, pf); break;
    case DType::F16: unscale_kernel<__half><<<grid, kThreads, 0, st>>>(g.data_as<__half>(), o.data_as<float>(), n, inv, pf); break;
    case DType::BF16: unscale_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(g.data_as<__nv_bfloat16>(), o.data_as<float>(), n, inv, pf); break;
    default: throw std::invalid_argument("amp unscale: gradients must be float32/float16/bfloat16");
  }
  check_launch("amp_unscale");
  c.i[0] = shared_flag ? 1 : (read_flag(flag, st) ? 0 : 1);
}

void k_amp_copy(OpCall& c) {
  Tensor& model = c.in[0];
  const Tensor& master = c.in[1];
  if (!model.is_contiguous() || !master.is_contiguous()) throw std::invalid_argument("amp copy: tensors must be contiguous on CUDA");
  const int64_t n = model.numel();
  const int grid = ew_grid(n, kThreads, sm_count_for(model));
  cudaStream_t st = stream_of(c);
  switch (model.dtype()) {
    case DType::F32: amp_copy_kernel<float><<<grid, kThreads, 0, st>>>(model.data_as<float>(), master.data_as<float>(), n); break;
    case DType::F16: amp_copy_kernel<__half><<<grid, kThreads, 0, st>>>(model.data_as<__half>(), master.data_as<float>(), n); break;
    case DType::BF16: amp_copy_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(model.data_as<__nv_bfloat16>(), master.data_as<float>(), n); break;
    default: throw std::invalid_argument("amp copy: model dtype must be float32/float16/bfloat16");
  }
  check_launch("amp_copy");
}

template <class G>
void adam_with_grad(OpCall& c) {
  Tensor &p = c.in[0], &m = c.in[1], &v = c.in[2];
  const Tensor& g = c.in[3];
  const AdamArgs a{static_cast<float>(c.f[0]), static_cast<float>(c.f[1]), static_cast<float>(c.f[2]), static_cast<float>(c.f[3]),
                   static_cast<float>(c.f[4]), static_cast<float>(1.0 / c.f[5]), static_cast<float>(1.0 / c.f[6]),
                   static_cast<float>(c.f[7])};
  const int64_t n = p.numel();
  cudaStream_t st = stream_of(c);
  float *pp = p.data_as<float>(), *pm = m.data_as<float>(), *pv = v.data_as<float>();
  const G* pg = g.data_as<G>();
  void* pmodel = c.in[4].defined() ? c.in[4].data() : nullptr;
  // Bulk in 8-element vectors, the (at most 7-element) tail with the scalar kernel.
  const int64_t n8 = aligned16(pp, pm, pv, pg, pmodel) ? n / 8 : 0;
  const int64_t done = n8 * 8, rest = n - done;
  const int sms = sm_count_for(p);
  const int vt = c.i[0] > 0 ? static_cast<int>(c.i[0]) : kThreads;  // block size of the vector pass
  auto launch = [&](auto model_ptr) {
    using MT = std::remove_pointer_t<decltype(model_ptr)>;
    if (n8 > 0) {
      static const bool once = (prefer_max_shared_carveout(adam_vec_kernel<G, MT>), true);
      (void)once;
      adam_vec_kernel<G, MT><<<ew_grid(n8, vt, sms), vt, 0, st>>>(pp, pm, pv, pg, model_ptr, n8, a);
    }
    if (rest > 0)
      adam_kernel<G, MT><<<ew_grid(rest, kThreads, sms), kThreads, 0, st>>>(pp + done, pm + done, pv + done, pg + done,
                                                                           model_ptr ? model_ptr + done : model_ptr, rest, a);
  };
  if (!c.in[4].defined()) launch(static_cast<float*>(nullptr));
  else if (c.in[4].dtype() == DType::BF16) launch(c.in[4].data_as<__nv_bfloat16>());
  else if (c.in[4].dtype() == DType::F16) launch(c.in[4].data_as<__half>());
  else launch(c.in[4].data_as<float>());
  check_launch("adam_step");
}

void k_adam(OpCall& c) {
  switch (c.in[3].dtype()) {
    case DType::F32: adam_with_grad<float>(c); break;
    case DType::F16: adam_with_grad<__half>(c); break;
    case DType::BF16: adam_with_grad<__nv_bfloat16>(c); break;
    default: throw std::invalid_argument("adam_step: gradient dtype must be float32/float16/bfloat16");
  }
}

template <class G>
void sgd_with_grad(OpCall& c) {
  Tensor& p = c.in[0];
  const Tensor& g = c.in[1];
  const int64_t n = p.numel();
  cudaStream_t st = stream_of(c);
  const float lr = static_cast<float>(c.f[0]), wd = static_cast<float>(c.f[1]), gs = static_cast<float>(c.f[2]);
  float* pp = p.data_as<float>();
  const G* pg = g.data_as<G>();
  void* pmodel = c.in[2].defined() ? c.in[2].data() : nullptr;
  const int64_t n8 = aligned16(pp, pg, pmodel) ? n / 8 : 0;
  const int64_t done = n8 * 8, rest = n - done;
  const int sms = sm_count_for(p);
  const int vt = c.i[0] > 0 ? static_cast<int>(c.i[0]) : kThreads;  // block size of the vector pass
  auto launch = [&](auto model_ptr) {
    using MT = std::remove_pointer_t<decltype(model_ptr)>;
    if (n8 > 0) {
      static const bool once = (prefer_max_shared_carveout(sgd_vec_kernel<G, MT>), true);
      (void)once;
      sgd_vec_kernel<G, MT><<<ew_grid(n8, vt, sms), vt, 0, st>>>(pp, pg, model_ptr, n8, lr, wd, gs);
    }
    if (rest > 0)
      sgd_kernel<G, MT><<<ew_grid(rest, kThreads, sms), kThreads, 0, st>>>(pp + done, pg + done, model_ptr ? model_ptr + done : model_ptr,
                                                                          rest, lr, wd, gs);
  };
  if (!c.in[2].defined()) launch(static_cast<float*>(nullptr));
  else if (c.in[2].dtype() == DType::BF16) launch(c.in[2].data_as<__nv_bfloat16>());
  else if (c.in[2].dtype() == DType::F16) launch(c.in[2].data_as<__half>());
  else launch(c.in[2].data_as<float>());
  check_launch("sgd_step");
}

void k_sgd(OpCall& c) {
  switch (c.in[1].dtype()) {
    case DType::F32: sgd_with_grad<float>(c); break;
    case DType::F16: sgd_with_grad<__half>(c); break;
    case DType::BF16: sgd_with_grad<__nv_bfloat16>(c); break;
    default: throw std::invalid_argument("sgd_step: gradient dtype must be float32/float16/bfloat16");
  }
}

}  // namespace

void register_cuda_elementwise(KernelRegistry& r) {
  const uint8_t any = kContiguous | kStrided | kEmpty;
#define REG3(OP, FN, NAME)                                                                                      \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, kMaskF32, any, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::F16), any, Capability::None}, FN<__half>, NAME "_f16"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::BF16), any, Capability::Bf16}, FN<__nv_bfloat16>, NAME "_bf16");
  REG3(Add, k_add, "sm100_add") REG3(Mul, k_mul, "sm100_mul")
  REG3(AddInplace, k_add_inplace, "sm100_add_") REG3(MulInplace, k_mul_inplace, "sm100_mul_")
  REG3(AddScalar, k_add_scalar, "sm100_add_scalar") REG3(MulScalar, k_mul_scalar, "sm100_mul_scalar")
  REG3(Neg, k_neg, "sm100_neg") REG3(Relu, k_relu, "sm100_relu") REG3(Sigmoid, k_sigmoid, "sm100_sigmoid")
  REG3(Tanh, k_tanh, "sm100_tanh") REG3(LeakyRelu, k_leaky, "sm100_leaky_relu") REG3(Gelu, k_gelu, "sm100_gelu")
  REG3(Exp, k_exp, "sm100_exp") REG3(Sqrt, k_sqrt, "sm100_sqrt") REG3(Reciprocal, k_recip, "sm100_reciprocal")
  REG3(Log, k_log, "sm100_log")
  REG3(ReluBackward, k_relu_b, "sm100_relu_backward") REG3(SigmoidBackward, k_sigmoid_b, "sm100_sigmoid_backward")
  REG3(TanhBackward, k_tanh_b, "sm100_tanh_backward") REG3(LeakyReluBackward, k_leaky_b, "sm100_leaky_relu_backward")
  REG3(GeluBackward, k_gelu_b, "sm100_gelu_backward") REG3(ExpBackward, k_exp_b, "sm100_exp_backward")
  REG3(SqrtBackward, k_sqrt_b, "sm100_sqrt_backward") REG3(ReciprocalBackward, k_recip_b, "sm100_reciprocal_backward")
  REG3(DropoutMask, k_dropout_mask, "sm100_dropout_mask")
#undef REG3
  r.add_kernel(OperatorId::Contiguous, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, k_contiguous, "sm100_strided_copy");
  r.add_kernel(OperatorId::Cast, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, k_cast, "sm100_cast");
  r.add_kernel(OperatorId::Fill, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, k_fill, "sm100_fill");
  r.add_kernel(OperatorId::CopyRange, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, k_copy_range, "sm100_copy_range");
  r.add_kernel(OperatorId::IsFiniteAll, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, k_isfinite, "sm100_isfinite_all");
  r.add_kernel(OperatorId::AmpUnscale, Constraints{Backend::CUDA, kMaskCudaCompute, any, Capability::None}, k_amp_unscale, "sm100_amp_unscale");
  r.add_kernel(OperatorId::AmpCopy, Constraints{Backend::CUDA, kMaskCudaCompute, any, Capability::None}, k_amp_copy, "sm100_amp_copy");
  r.add_kernel(OperatorId::AdamStep, Constraints{Backend::CUDA, kMaskF32, kContiguous | kEmpty, Capability::None}, k_adam, "sm100_adam_step");
  r.add_kernel(OperatorId::SgdStep, Constraints{Backend::CUDA, kMaskF32, kContiguous | kEmpty, Capability::None}, k_sgd, "sm100_sgd_step");
}

}  // namespace cu
}  // namespace ob

// CPU reference backend, part 1: elementwise, casts, copies, fills and reductions.
// These kernels are the numerical oracle for the sm_100a kernels; they favour clarity
// (stride walking, double accumulators for full reductions) over speed.
//
// Parity (reference project paths): src/backends/cpu/{binary,unary,cast,fill,copy,
// reduce,unbroadcast,max_backward,tensor_access}.cpp.
#include <cmath>
#include <cstring>
#include <limits>

#include "ob/kernels.h"

namespace ob {
namespace {

// Walks every element of `shape` in row-major order and reports the element offsets of
// up to three operands with their own strides.
template <class F>
void walk(const Shape& shape, const Shape& s0, const Shape& s1, const Shape& s2, F&& f) {
  const int nd = static_cast<int>(shape.size());
  int64_t total = 1;
  for (int64_t d : shape) total *= d;
  if (total == 0) return;
  std::vector<int64_t> idx(nd, 0);
  int64_t o0 = 0, o1 = 0, o2 = 0;
  for (int64_t n = 0; n < total; ++n) {
    f(o0, o1, o2);
    for (int d = nd - 1; d >= 0; --d) {
      ++idx[d];
      o0 += s0.empty() ? 0 : s0[d];
      o1 += s1.empty() ? 0 : s1[d];
      o2 += s2.empty() ? 0 : s2[d];
      if (idx[d] < shape[d]) break;
      o0 -= s0.empty() ? 0 : s0[d] * shape[d];
      o1 -= s1.empty() ? 0 : s1[d] * shape[d];
      o2 -= s2.empty() ? 0 : s2[d] * shape[d];
      idx[d] = 0;
    }
  }
}

// Strides of `t` aligned to `out_shape` with 0 where `t` is broadcast.
Shape broadcast_strides(const Tensor& t, const Shape& out_shape) {
  const int nd = static_cast<int>(out_shape.size());
  const int td = t.ndim();
  Shape st(nd, 0);
  for (int i = 0; i < td; ++i) {
    const int o = nd - td + i;
    st[o] = (t.shape()[i] == 1 && out_shape[o] != 1) ? 0 : t.strides()[i];
  }
  return st;
}

template <class T, class Op>
void binary_kernel(OpCall& c, Op op) {
  const Tensor &a = c.in[0], &b = c.in[1];
  Tensor& out = c.out[0];
  const T* pa = a.data_as<T>();
  const T* pb = b.data_as<T>();
  T* po = out.data_as<T>();
  if (a.is_contiguous() && b.is_contiguous() && a.shape() == out.shape() && b.shape() == out.shape()) {
    const int64_t n = out.numel();
    for (int64_t i = 0; i < n; ++i) po[i] = op(pa[i], pb[i]);
    return;
  }
  walk(out.shape(), out.strides(), broadcast_strides(a, out.shape()), broadcast_strides(b, out.shape()),
       [&](int64_t o, int64_t ia, int64_t ib) { po[o] = op(pa[ia], pb[ib]); });
}

template <class T> void add_cpu(OpCall& c) { binary_kernel<T>(c, [](T x, T y) { return x + y; }); }
template <class T> void mul_cpu(OpCall& c) { binary_kernel<T>(c, [](T x, T y) { return x * y; }); }

template <class T>
void add_inplace_cpu(OpCall& c) {
  Tensor& a = c.in[0];
  const Tensor& b = c.in[1];
  const T alpha = static_cast<T>(c.f[0]);
  T* pa = a.data_as<T>();
  const T* pb = b.data_as<T>();
  walk(a.shape(), a.strides(), broadcast_strides(b, a.shape()), {},
       [&](int64_t ia, int64_t ib, int64_t) { pa[ia] += alpha * pb[ib]; });
}

template <class T>
void mul_inplace_cpu(OpCall& c) {
  Tensor& a = c.in[0];
  const T alpha = static_cast<T>(c.f[0]);
  T* pa = a.data_as<T>();
  walk(a.shape(), a.strides(), {}, {}, [&](int64_t ia, int64_t, int64_t) { pa[ia] *= alpha; });
}

template <class T, class Op>
void map_kernel(OpCall& c, Op op) {
  const Tensor& a = c.in[0];
  Tensor& out = c.out[0];
  const T* pa = a.data_as<T>();
  T* po = out.data_as<T>();
  if (a.is_contiguous()) {
    const int64_t n = out.numel();
    for (int64_t i = 0; i < n; ++i) po[i] = op(pa[i]);
    return;
  }
  walk(out.shape(), out.strides(), a.strides(), {}, [&](int64_t o, int64_t ia, int64_t) { po[o] = op(pa[ia]); });
}

template <class T, class Op>
void map2_kernel(OpCall& c, Op op) {  // out = op(x, grad)
  const Tensor &x = c.in[0], &g = c.in[1];
  Tensor& out = c.out[0];
  const T* px = x.data_as<T>();
  const T* pg = g.data_as<T>();
  T* po = out.data_as<T>();
  walk(out.shape(), out.strides(), x.strides(), g.strides(),
       [&](int64_t o, int64_t ix, int64_t ig) { po[o] = op(px[ix], pg[ig]); });
}

template <class T> void add_scalar_cpu(OpCall& c) { const T s = static_cast<T>(c.f[0]); map_kernel<T>(c, [s](T x) { return x + s; }); }
template <class T> void mul_scalar_cpu(OpCall& c) { const T s = static_cast<T>(c.f[0]); map_kernel<T>(c, [s](T x) { return x * s; }); }
template <class T> void neg_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return -x; }); }
template <class T> void relu_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return x > T(0) ? x : T(0); }); }
template <class T> void sigmoid_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return T(1) / (T(1) + std::exp(-x)); }); }
template <class T> void tanh_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return std::tanh(x); }); }
template <class T> void leaky_cpu(OpCall& c) { const T s = static_cast<T>(c.f[0]); map_kernel<T>(c, [s](T x) { return x > T(0) ? x : s * x; }); }
template <class T> void gelu_cpu(OpCall& c) {
  map_kernel<T>(c, [](T x) { return T(0.5) * x * (T(1) + std::erf(x * T(0.70710678118654752440))); });
}
template <class T> void exp_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return std::exp(x); }); }
template <class T> void sqrt_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return std::sqrt(x); }); }
template <class T> void recip_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return T(1) / x; }); }
template <class T> void log_cpu(OpCall& c) { map_kernel<T>(c, [](T x) { return std::log(x); }); }

template <class T> void relu_bwd_cpu(OpCall& c) { map2_kernel<T>(c, [](T x, T g) { return x > T(0) ? g : T(0); }); }
template <class T> void sigmoid_bwd_cpu(OpCall& c) {
  map2_kernel<T>(c, [](T x, T g) { const T s = T(1) / (T(1) + std::exp(-x)); return g * s * (T(1) - s); });
}
template <class T> void tanh_bwd_cpu(OpCall& c) {
  map2_kernel<T>(c, [](T x, T g) { const T t = std::tanh(x); return g * (T(1) - t * t); });
}
template <class T> void leaky_bwd_cpu(OpCall& c) {
  const T s = static_cast<T>(c.f[0]);
  map2_kernel<T>(c, [s](T x, T g) { return x > T(0) ? g : s * g; });
}
template <class T> void gelu_bwd_cpu(OpCall& c) {
  map2_kernel<T>(c, [](T x, T g) {
    const T cdf = T(0.5) * (T(1) + std::erf(x * T(0.70710678118654752440)));
    const T pdf = T(0.39894228040143267794) * std::exp(T(-0.5) * x * x);
    return g * (cdf + x * pdf);
  });
}
template <class T> void exp_bwd_cpu(OpCall& c) { map2_kernel<T>(c, [](T x, T g) { return g * std::exp(x); }); }
template <class T> void sqrt_bwd_cpu(OpCall& c) { map2_kernel<T>(c, [](T x, T g) { return g / (T(2) * std::sqrt(x)); }); }
template <class T> void recip_bwd_cpu(OpCall& c) { map2_kernel<T>(c, [](T x, T g) { return -g / (x * x); }); }

// -------------------------------------------------------------- copies and casts
void contiguous_cpu(OpCall& c) {  // strided -> strided copy, any dtype
  const Tensor& src = c.in[0];
  Tensor& dst = c.out[0];
  const size_t esz = dtype_size(src.dtype());
  const char* ps = static_cast<const char*>(src.data());
  char* pd = static_cast<char*>(dst.data());
  if (src.is_contiguous() && dst.is_contiguous()) {
    if (src.numel()) std::memcpy(pd, ps, src.nbytes());
    return;
  }
  walk(dst.shape(), dst.strides(), broadcast_strides(src, dst.shape()), {},
       [&](int64_t o, int64_t i, int64_t) { std::memcpy(pd + o * esz, ps + i * esz, esz); });
}

void cast_cpu(OpCall& c) {  // all 81 pairs through double
  const Tensor& src = c.in[0];
  Tensor& dst = c.out[0];
  const size_t es = dtype_size(src.dtype()), ed = dtype_size(dst.dtype());
  const char* ps = static_cast<const char*>(src.data());
  char* pd = static_cast<char*>(dst.data());
  const DType sd = src.dtype(), dd = dst.dtype();
  walk(dst.shape(), dst.strides(), src.strides(), {}, [&](int64_t o, int64_t i, int64_t) {
    if (sd == DType::I64 && dd == DType::I64) {
      std::memcpy(pd + o * ed, ps + i * es, 8);
    } else if (sd == DType::I64 && (dd == DType::I32 || dd == DType::I8 || dd == DType::U8 || dd == DType::Bool)) {
      int64_t v; std::memcpy(&v, ps + i * es, 8);
      if (dd == DType::I32) { int32_t x = static_cast<int32_t>(v); std::memcpy(pd + o * ed, &x, 4); }
      else if (dd == DType::I8) { *reinterpret_cast<int8_t*>(pd + o) = static_cast<int8_t>(v); }
      else if (dd == DType::U8) { *reinterpret_cast<uint8_t*>(pd + o) = static_cast<uint8_t>(v); }
      else { *reinterpret_cast<uint8_t*>(pd + o) = v != 0; }
    } else {
      store_from_double(pd + o * ed, dd, load_as_double(ps + i * es, sd));
    }
  });
}

void fill_cpu(OpCall& c) {
  Tensor& t = c.in[0];
  const size_t esz = dtype_size(t.dtype());
  char one[8];
  store_from_double(one, t.dtype(), c.f[0]);
  char* p = static_cast<char*>(t.data());
  if (t.is_contiguous()) {
    const int64_t n = t.numel();
    bool zero = true;
    for (size_t i = 0; i < esz; ++i) zero = zero && one[i] == 0;
    if (zero) { if (n) std::memset(p, 0, n * esz); return; }
    for (int64_t i = 0; i < n; ++i) std::memcpy(p + i * esz, one, esz);
    return;
  }
  walk(t.shape(), t.strides(), {}, {}, [&](int64_t o, int64_t, int64_t) { std::memcpy(p + o * esz, one, esz); });
}

void copy_range_cpu(OpCall& c) {
  Tensor& dst = c.in[0];
  const Tensor& src = c.in[1];
  const size_t esz = dtype_size(dst.dtype());
  if (c.i[2] > 0)
    std::memcpy(static_cast<char*>(dst.data()) + c.i[0] * esz, static_cast<const char*>(src.data()) + c.i[1] * esz,
                c.i[2] * esz);
}


void isfinite_cpu(OpCall& c) {
  const Tensor& t = c.in[0];
  c.i[0] = 1;
  if (!dtype_is_floating(t.dtype())) return;
  const size_t esz = dtype_size(t.dtype());
  const char* p = static_cast<const char*>(t.data());
  bool ok = true;
  walk(t.shape(), t.strides(), {}, {}, [&](int64_t o, int64_t, int64_t) {
    if (!std::isfinite(load_as_double(p + o * esz, t.dtype()))) ok = false;
  });
  if (c.in[1].defined() && !ok) c.in[1].data_as<int32_t>()[0] = 1;
  c.i[0] = ok ? 1 : 0;
}

void amp_unscale_cpu(OpCall& c) {
  const Tensor& g = c.in[0];
  Tensor& out = c.out[0];
  const float inv = static_cast<float>(c.f[0]);
  const size_t esz = dtype_size(g.dtype());
  const char* p = static_cast<const char*>(g.data());
  float* po = out.data_as<float>();
  bool ok = true;
  walk(out.shape(), out.strides(), g.strides(), {}, [&](int64_t o, int64_t i, int64_t) {
    const float v = static_cast<float>(load_as_double(p + i * esz, g.dtype())) * inv;
    if (!std::isfinite(v)) ok = false;
    po[o] = v;
  });
  if (c.in[1].defined() && !ok) c.in[1].data_as<int32_t>()[0] = 1;
  c.i[0] = ok ? 1 : 0;
}

void amp_copy_cpu(OpCall& c) {
  Tensor& model = c.in[0];
  const Tensor& master = c.in[1];
  const size_t esz = dtype_size(model.dtype());
  char* pd = static_cast<char*>(model.data());
  const float* ps = master.data_as<float>();
  walk(model.shape(), model.strides(), master.strides(), {},
       [&](int64_t o, int64_t i, int64_t) { store_from_double(pd + o * esz, model.dtype(), ps[i]); });
}

// ------------------------------------------------------------------ reductions
template <class T>
void sum_cpu_impl(OpCall& c, bool mean) {
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* p = c.in[0].data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) {
      double acc = 0.0;
      for (int64_t r = 0; r < red; ++r) acc += p[(o * red + r) * inner + k];
      po[o * inner + k] = static_cast<T>(mean ? acc / static_cast<double>(red) : acc);
    }
}
template <class T> void sum_cpu(OpCall& c) { sum_cpu_impl<T>(c, false); }
template <class T> void mean_cpu(OpCall& c) { sum_cpu_impl<T>(c, true); }

template <class T>
void max_cpu(OpCall& c) {
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* p = c.in[0].data_as<T>();
  T* pv = c.out[0].data_as<T>();
  int64_t* pi = c.out[1].data_as<int64_t>();
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) {
      T best = p[(o * red) * inner + k];
      int64_t bi = 0;
      for (int64_t r = 1; r < red; ++r) {
        const T v = p[(o * red + r) * inner + k];
        if (extrema_better(v, best)) { best = v; bi = r; }
      }
      pv[o * inner + k] = best;
      pi[o * inner + k] = bi;
    }
}

template <class T>
void max_backward_cpu(OpCall& c) {
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* pg = c.in[0].data_as<T>();
  const int64_t* pi = c.in[1].data_as<int64_t>();
  T* po = c.out[0].data_as<T>();
  std::memset(po, 0, sizeof(T) * outer * red * inner);
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) po[(o * red + pi[o * inner + k]) * inner + k] = pg[o * inner + k];
}

template <class T>
void unbroadcast_cpu(OpCall& c) {
  const Tensor& g = c.in[0];
  Tensor& out = c.out[0];
  const Shape& padded = c.list;  // target shape padded to g's rank
  Shape ost(padded.size(), 0);
  int64_t run = 1;
  for (int i = static_cast<int>(padded.size()) - 1; i >= 0; --i) {
    ost[i] = (padded[i] == 1 && g.shape()[i] != 1) ? 0 : run;
    run *= padded[i];
  }
  const T* pg = g.data_as<T>();
  T* po = out.data_as<T>();
  std::vector<double> acc(static_cast<size_t>(out.numel()), 0.0);
  walk(g.shape(), g.strides(), ost, {}, [&](int64_t ig, int64_t io, int64_t) { acc[io] += pg[ig]; });
  for (int64_t i = 0; i < out.numel(); ++i) po[i] = static_cast<T>(acc[i]);
}

void dropout_mask_cpu(OpCall& c) {
  Tensor& out = c.out[0];
  const float p = static_cast<float>(c.f[0]);
  const float scale = 1.0f / (1.0f - p);
  const uint64_t seed = static_cast<uint64_t>(c.i[0]);
  const int64_t n = out.numel();
  const size_t esz = dtype_size(out.dtype());
  char* po = static_cast<char*>(out.data());
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t top24 = static_cast<uint32_t>(splitmix64(seed + static_cast<uint64_t>(i)) >> 40);
    const float r = static_cast<float>(top24) * (1.0f / 16777216.0f);
    store_from_double(po + i * esz, out.dtype(), r >= p ? scale : 0.0f);
  }
}

}  // namespace

void register_cpu_elementwise(KernelRegistry& r) {
  const uint8_t any = kContiguous | kStrided | kEmpty;
#define REG2(OP, FN, NAME)                                                                          \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CPU, kMaskF32, any, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CPU, kMaskF64, any, Capability::None}, FN<double>, NAME "_f64");
  REG2(Add, add_cpu, "cpu_add") REG2(Mul, mul_cpu, "cpu_mul")
  REG2(AddInplace, add_inplace_cpu, "cpu_add_") REG2(MulInplace, mul_inplace_cpu, "cpu_mul_")
  REG2(AddScalar, add_scalar_cpu, "cpu_add_scalar") REG2(MulScalar, mul_scalar_cpu, "cpu_mul_scalar")
  REG2(Neg, neg_cpu, "cpu_neg") REG2(Relu, relu_cpu, "cpu_relu") REG2(Sigmoid, sigmoid_cpu, "cpu_sigmoid")
  REG2(Tanh, tanh_cpu, "cpu_tanh") REG2(LeakyRelu, leaky_cpu, "cpu_leaky_relu") REG2(Gelu, gelu_cpu, "cpu_gelu")
  REG2(Exp, exp_cpu, "cpu_exp") REG2(Sqrt, sqrt_cpu, "cpu_sqrt") REG2(Reciprocal, recip_cpu, "cpu_reciprocal")
  REG2(Log, log_cpu, "cpu_log")
  REG2(ReluBackward, relu_bwd_cpu, "cpu_relu_backward") REG2(SigmoidBackward, sigmoid_bwd_cpu, "cpu_sigmoid_backward")
  REG2(TanhBackward, tanh_bwd_cpu, "cpu_tanh_backward") REG2(LeakyReluBackward, leaky_bwd_cpu, "cpu_leaky_relu_backward")
  REG2(GeluBackward, gelu_bwd_cpu, "cpu_gelu_backward") REG2(ExpBackward, exp_bwd_cpu, "cpu_exp_backward")
  REG2(SqrtBackward, sqrt_bwd_cpu, "cpu_sqrt_backward") REG2(ReciprocalBackward, recip_bwd_cpu, "cpu_reciprocal_backward")
  REG2(Sum, sum_cpu, "cpu_sum") REG2(Mean, mean_cpu, "cpu_mean") REG2(Max, max_cpu, "cpu_max")
  REG2(MaxBackward, max_backward_cpu, "cpu_max_backward") REG2(Unbroadcast, unbroadcast_cpu, "cpu_unbroadcast")
#undef REG2
  r.add_kernel(OperatorId::Contiguous, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, contiguous_cpu, "cpu_strided_copy");
  r.add_kernel(OperatorId::Cast, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, cast_cpu, "cpu_cast");
  r.add_kernel(OperatorId::Fill, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, fill_cpu, "cpu_fill");
  r.add_kernel(OperatorId::CopyRange, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, copy_range_cpu, "cpu_copy_range");
  r.add_kernel(OperatorId::IsFiniteAll, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, isfinite_cpu, "cpu_isfinite_all");
  r.add_kernel(OperatorId::AmpUnscale, Constraints{Backend::CPU, kMaskF32 | kMaskF64 | kMaskHalf, any, Capability::None}, amp_unscale_cpu, "cpu_amp_unscale");
  r.add_kernel(OperatorId::AmpCopy, Constraints{Backend::CPU, kMaskF32 | kMaskHalf, any, Capability::None}, amp_copy_cpu, "cpu_amp_copy");
  r.add_kernel(OperatorId::DropoutMask, Constraints{Backend::CPU, kMaskF32 | kMaskF64 | kMaskHalf, any, Capability::None}, dropout_mask_cpu, "cpu_dropout_mask");
}

}  // namespace ob

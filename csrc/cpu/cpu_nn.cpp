// CPU reference backend, part 2: matmul, softmax family, losses, embedding, conv2d,
// maxpool, LayerNorm, causal softmax and the optimizer update formulas.
//
// Parity (reference project paths): src/backends/cpu/{matmul,softmax,cross_entropy,
// nll_loss,embedding,conv2d,maxpool2d,fusion}.cpp; optimizer math from
// python/orthon/optim/adam.py:134-183 and python/orthon/optim/sgd.py:35-42.
#include <cmath>
#include <cstring>
#include <limits>

#include "ob/cpu_parallel.h"
#include "ob/kernels.h"

namespace ob {
namespace {

inline int64_t target_at(const Tensor& t, int64_t i) {
  return t.dtype() == DType::I64 ? t.data_as<int64_t>()[i] : static_cast<int64_t>(t.data_as<int32_t>()[i]);
}

// Vector kernels of the matmul family.  Written as plain loops over contiguous arrays so the
// compiler vectorises them; clones for wider vector ISAs are selected at load time.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define OB_VEC_CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))
#else
#define OB_VEC_CLONES
#endif

#define OB_DEFINE_VEC_KERNELS(T, SUFFIX)                                                             \
  OB_VEC_CLONES void axpy_##SUFFIX(T* __restrict__ c, const T* __restrict__ b, T a, int64_t n) {     \
    for (int64_t j = 0; j < n; ++j) c[j] += a * b[j];                                                \
  }                                                                                                  \
  OB_VEC_CLONES T dot_##SUFFIX(const T* __restrict__ a, const T* __restrict__ b, int64_t n) {        \
    T acc[16] = {};                                                                                  \
    int64_t k = 0;                                                                                   \
    for (; k + 16 <= n; k += 16)                                                                     \
      for (int l = 0; l < 16; ++l) acc[l] += a[k + l] * b[k + l];                                    \
    T s = T(0);                                                                                      \
    for (; k < n; ++k) s += a[k] * b[k];                                                             \
    for (int l = 0; l < 16; ++l) s += acc[l];                                                        \
    return s;                                                                                        \
  }
OB_DEFINE_VEC_KERNELS(float, f32)
OB_DEFINE_VEC_KERNELS(double, f64)
#undef OB_DEFINE_VEC_KERNELS

inline void axpy(float* c, const float* b, float a, int64_t n) { axpy_f32(c, b, a, n); }
inline void axpy(double* c, const double* b, double a, int64_t n) { axpy_f64(c, b, a, n); }
inline float dot(const float* a, const float* b, int64_t n) { return dot_f32(a, b, n); }
inline double dot(const double* a, const double* b, int64_t n) { return dot_f64(a, b, n); }

// One batch entry: C[M, N] = A'[M, K] @ B'[K, N] through element strides.  Rows of C are split
// over the worker pool; every element is produced by one worker in a fixed order.
template <class T>
void gemm_rows(const T* pa, int64_t a_rs, int64_t a_cs, const T* pb, int64_t b_rs, int64_t b_cs, T* pc, int64_t c_rs,
               int64_t c_cs, int64_t M, int64_t N, int64_t K) {
  const int64_t work_per_row = std::max<int64_t>(1, N * K);
  const int64_t grain = std::max<int64_t>(1, (1 << 16) / work_per_row);
  cpu::parallel_for(M, grain, [&](int64_t lo, int64_t hi) {
    if (b_cs == 1 && c_cs == 1) {
      // B rows contiguous: accumulate row i of C as a sum of scaled rows of B.
      for (int64_t i = lo; i < hi; ++i) {
        T* crow = pc + i * c_rs;
        for (int64_t j = 0; j < N; ++j) crow[j] = T(0);
        for (int64_t k = 0; k < K; ++k) axpy(crow, pb + k * b_rs, pa[i * a_rs + k * a_cs], N);
      }
    } else if (b_rs == 1 && a_cs == 1) {
      // Both operands contiguous along K (B given transposed): dot products.
      for (int64_t i = lo; i < hi; ++i)
        for (int64_t j = 0; j < N; ++j) pc[i * c_rs + j * c_cs] = dot(pa + i * a_rs, pb + j * b_cs, K);
    } else {
      for (int64_t i = lo; i < hi; ++i) {
        for (int64_t j = 0; j < N; ++j) pc[i * c_rs + j * c_cs] = T(0);
        for (int64_t k = 0; k < K; ++k) {
          const T av = pa[i * a_rs + k * a_cs];
          for (int64_t j = 0; j < N; ++j) pc[i * c_rs + j * c_cs] += av * pb[k * b_rs + j * b_cs];
        }
      }
    }
  });
}

// C[b] = op(A[b]) @ op(B[b]); operands addressed through element strides, so transposed
// and sliced views need no packing.
template <class T>
void matmul_cpu(OpCall& c) {
  const Tensor &A = c.in[0], &B = c.in[1];
  Tensor& C = c.out[0];
  const bool ta = c.i[0] != 0, tb = c.i[1] != 0;
  const int r = A.ndim() - 2;  // number of batch dims (0, 1 or 2)
  const int64_t nb1 = r >= 1 ? A.shape()[r - 1] : 1;
  const int64_t nb0 = r >= 2 ? A.shape()[0] : 1;
  int64_t a_rs = A.strides()[r], a_cs = A.strides()[r + 1], b_rs = B.strides()[r], b_cs = B.strides()[r + 1];
  int64_t M = A.shape()[r], K = A.shape()[r + 1], N = B.shape()[r + 1];
  if (ta) { std::swap(a_rs, a_cs); std::swap(M, K); }
  if (tb) { std::swap(b_rs, b_cs); N = B.shape()[r]; }
  const int64_t c_rs = C.strides()[r], c_cs = C.strides()[r + 1];
  auto bstride = [r](const Tensor& t, int which) -> int64_t {  // which: 0 = outer batch, 1 = inner batch
    if (r == 2) return t.strides()[which];
    if (r == 1 && which == 1) return t.strides()[0];
    return 0;
  };
  for (int64_t bb = 0; bb < nb0 * nb1; ++bb) {
    const int64_t b0 = bb / nb1, b1 = bb % nb1;
    const T* pa = A.data_as<T>() + b0 * bstride(A, 0) + b1 * bstride(A, 1);
    const T* pb = B.data_as<T>() + b0 * bstride(B, 0) + b1 * bstride(B, 1);
    T* pc = C.data_as<T>() + b0 * bstride(C, 0) + b1 * bstride(C, 1);
    gemm_rows<T>(pa, a_rs, a_cs, pb, b_rs, b_cs, pc, c_rs, c_cs, M, N, K);
  }
}

template <class T>
void linear_cpu(OpCall& c) {
  const Tensor &x = c.in[0], &w = c.in[1], &bias = c.in[2], &res = c.in[3];
  Tensor& y = c.out[0];
  const int act = static_cast<int>(c.i[0]);
  const int64_t M = x.shape()[0], K = x.shape()[1], N = w.shape()[1];
  const T* px = x.data_as<T>();
  const T* pw = w.data_as<T>();
  T* py = y.data_as<T>();
  T* pz = c.out[1].defined() ? c.out[1].data_as<T>() : nullptr;
  const int64_t x_rs = x.strides()[0], x_cs = x.strides()[1], w_rs = w.strides()[0], w_cs = w.strides()[1];
  const int64_t grain = std::max<int64_t>(1, (1 << 16) / std::max<int64_t>(1, N * K));
  cpu::parallel_for(M, grain, [&](int64_t lo, int64_t hi) {
    std::vector<T> row(static_cast<size_t>(N));
    for (int64_t i = lo; i < hi; ++i) {
      for (int64_t j = 0; j < N; ++j) row[j] = bias.defined() ? bias.data_as<T>()[j] : T(0);
      if (w_cs == 1) {
        for (int64_t k = 0; k < K; ++k) axpy(row.data(), pw + k * w_rs, px[i * x_rs + k * x_cs], N);
      } else {
        for (int64_t k = 0; k < K; ++k) {
          const T xv = px[i * x_rs + k * x_cs];
          for (int64_t j = 0; j < N; ++j) row[j] += xv * pw[k * w_rs + j * w_cs];
        }
      }
      for (int64_t j = 0; j < N; ++j) {
        T v = row[j];
        if (pz)  // act 4 keeps the GELU derivative for the backward pass instead of the pre-activation
          pz[i * N + j] = act == 4 ? T(0.5) * (T(1) + std::erf(v * T(0.70710678118654752440))) +
                                         v * T(0.39894228040143267794) * std::exp(T(-0.5) * v * v)
                                   : v;
        if (act == 1) v = v > T(0) ? v : T(0);
        else if (act == 2 || act == 4) v = T(0.5) * v * (T(1) + std::erf(v * T(0.70710678118654752440)));
        if (res.defined()) {
          const T aux = res.data_as<T>()[i * N + j];
          v = act == 3 ? v * aux : v + aux;  // act 3: aux is a stored activation derivative
        }
        py[i * N + j] = v;
      }
    }
  });
}

template <class T>
void softmax_cpu_impl(OpCall& c, bool log_form) {
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* p = c.in[0].data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) {
      const T* base = p + o * red * inner + k;
      T* ob_ = po + o * red * inner + k;
      T mx = -std::numeric_limits<T>::infinity();
      for (int64_t r = 0; r < red; ++r) mx = std::max(mx, base[r * inner]);
      double s = 0.0;
      for (int64_t r = 0; r < red; ++r) s += std::exp(static_cast<double>(base[r * inner] - mx));
      const T ls = static_cast<T>(std::log(s));
      for (int64_t r = 0; r < red; ++r) {
        const T v = base[r * inner] - mx;
        ob_[r * inner] = log_form ? v - ls : static_cast<T>(std::exp(static_cast<double>(v)) / s);
      }
    }
}
template <class T> void softmax_cpu(OpCall& c) { softmax_cpu_impl<T>(c, false); }
template <class T> void log_softmax_cpu(OpCall& c) { softmax_cpu_impl<T>(c, true); }

template <class T>
void softmax_bwd_cpu(OpCall& c) {  // dx = y * (g - sum(g*y))
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* py = c.in[0].data_as<T>();
  const T* pg = c.in[1].data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) {
      const int64_t b = o * red * inner + k;
      double dot = 0.0;
      for (int64_t r = 0; r < red; ++r) dot += static_cast<double>(py[b + r * inner]) * pg[b + r * inner];
      for (int64_t r = 0; r < red; ++r)
        po[b + r * inner] = py[b + r * inner] * (pg[b + r * inner] - static_cast<T>(dot));
    }
}

template <class T>
void log_softmax_bwd_cpu(OpCall& c) {  // dx = g - exp(y) * sum(g)
  const int64_t outer = c.i[0], red = c.i[1], inner = c.i[2];
  const T* py = c.in[0].data_as<T>();
  const T* pg = c.in[1].data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < inner; ++k) {
      const int64_t b = o * red * inner + k;
      double s = 0.0;
      for (int64_t r = 0; r < red; ++r) s += pg[b + r * inner];
      for (int64_t r = 0; r < red; ++r)
        po[b + r * inner] = pg[b + r * inner] - static_cast<T>(std::exp(static_cast<double>(py[b + r * inner])) * s);
    }
}

template <class T>
void cross_entropy_cpu(OpCall& c) {
  const Tensor& logits = c.in[0];
  const int64_t B = logits.shape()[0], C = logits.shape()[1];
  const T* p = logits.data_as<T>();
  float* lse = c.out[1].data_as<float>();
  double total = 0.0;
  for (int64_t i = 0; i < B; ++i) {
    const T* row = p + i * C;
    T mx = row[0];
    for (int64_t j = 1; j < C; ++j) mx = std::max(mx, row[j]);
    double s = 0.0;
    for (int64_t j = 0; j < C; ++j) s += std::exp(static_cast<double>(row[j] - mx));
    const double l = static_cast<double>(mx) + std::log(s);
    lse[i] = static_cast<float>(l);
    total += l - static_cast<double>(row[target_at(c.in[1], i)]);
  }
  store_from_double(c.out[0].data(), c.out[0].dtype(), total / static_cast<double>(B));
}

template <class T>
void cross_entropy_bwd_cpu(OpCall& c) {
  const Tensor& logits = c.in[0];
  const int64_t B = logits.shape()[0], C = logits.shape()[1];
  const T* p = logits.data_as<T>();
  const double g = load_as_double(c.in[2].data(), c.in[2].dtype()) / static_cast<double>(B);
  const float* lse = c.in[3].data_as<float>();
  T* po = c.out[0].data_as<T>();
  for (int64_t i = 0; i < B; ++i) {
    const int64_t t = target_at(c.in[1], i);
    for (int64_t j = 0; j < C; ++j) {
      const double sm = std::exp(static_cast<double>(p[i * C + j]) - lse[i]);
      po[i * C + j] = static_cast<T>((sm - (j == t ? 1.0 : 0.0)) * g);
    }
  }
}

template <class T>
void nll_cpu(OpCall& c) {
  const Tensor& lp = c.in[0];
  const int64_t N = lp.shape()[0], C = lp.shape()[1];
  const T* p = lp.data_as<T>();
  T* po = c.out[0].data_as<T>();
  const int red = static_cast<int>(c.i[0]);
  double total = 0.0;
  for (int64_t i = 0; i < N; ++i) {
    const T v = -p[i * C + target_at(c.in[1], i)];
    if (red == 0) po[i] = v;
    else total += v;
  }
  if (red == 1) po[0] = static_cast<T>(total / static_cast<double>(N));
  if (red == 2) po[0] = static_cast<T>(total);
}

template <class T>
void nll_bwd_cpu(OpCall& c) {
  Tensor& out = c.out[0];
  const int64_t N = out.shape()[0], C = out.shape()[1];
  const T* pg = c.in[0].data_as<T>();
  T* po = out.data_as<T>();
  const int red = static_cast<int>(c.i[0]);
  std::memset(po, 0, sizeof(T) * N * C);
  for (int64_t i = 0; i < N; ++i) {
    const T g = red == 0 ? pg[i] : (red == 1 ? pg[0] / static_cast<T>(N) : pg[0]);
    po[i * C + target_at(c.in[1], i)] = -g;
  }
}

template <class T>
void embedding_cpu(OpCall& c) {
  const Tensor &idx = c.in[0], &w = c.in[1];
  const int64_t n = idx.numel(), D = w.shape()[1];
  const T* pw = w.data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t i = 0; i < n; ++i) std::memcpy(po + i * D, pw + target_at(idx, i) * D, sizeof(T) * D);
}

template <class T>
void embedding_bwd_cpu(OpCall& c) {
  const Tensor &idx = c.in[0], &g = c.in[1];
  Tensor& dw = c.out[0];
  const int64_t n = idx.numel(), D = dw.shape()[1];
  T* po = dw.data_as<T>();
  std::memset(po, 0, sizeof(T) * dw.numel());
  const T* pg = g.data_as<T>();
  for (int64_t i = 0; i < n; ++i) {
    T* row = po + target_at(idx, i) * D;
    for (int64_t d = 0; d < D; ++d) row[d] += pg[i * D + d];
  }
}

struct ConvGeom {
  int64_t N, C, H, W, K, R, S, OH, OW, sh, sw, ph, pw;
};

ConvGeom conv_geom(const Shape& x, const Shape& w, const int64_t* i) {
  ConvGeom g;
  g.N = x[0]; g.C = x[1]; g.H = x[2]; g.W = x[3];
  g.K = w[0]; g.R = w[2]; g.S = w[3];
  g.sh = i[0]; g.sw = i[1]; g.ph = i[2]; g.pw = i[3];
  g.OH = (g.H + 2 * g.ph - g.R) / g.sh + 1;
  g.OW = (g.W + 2 * g.pw - g.S) / g.sw + 1;
  return g;
}

template <class T>
void conv2d_cpu(OpCall& c) {
  const ConvGeom g = conv_geom(c.in[0].shape(), c.in[1].shape(), c.i);
  const T* px = c.in[0].data_as<T>();
  const T* pw = c.in[1].data_as<T>();
  const T* pb = c.in[2].defined() ? c.in[2].data_as<T>() : nullptr;
  T* po = c.out[0].data_as<T>();
  for (int64_t n = 0; n < g.N; ++n)
    for (int64_t k = 0; k < g.K; ++k)
      for (int64_t oh = 0; oh < g.OH; ++oh)
        for (int64_t ow = 0; ow < g.OW; ++ow) {
          double acc = pb ? pb[k] : 0.0;
          for (int64_t ci = 0; ci < g.C; ++ci)
            for (int64_t r = 0; r < g.R; ++r) {
              const int64_t ih = oh * g.sh - g.ph + r;
              if (ih < 0 || ih >= g.H) continue;
              for (int64_t s = 0; s < g.S; ++s) {
                const int64_t iw = ow * g.sw - g.pw + s;
                if (iw < 0 || iw >= g.W) continue;
                acc += static_cast<double>(px[((n * g.C + ci) * g.H + ih) * g.W + iw]) *
                       pw[((k * g.C + ci) * g.R + r) * g.S + s];
              }
            }
          po[((n * g.K + k) * g.OH + oh) * g.OW + ow] = static_cast<T>(acc);
        }
}

template <class T>
void conv2d_bwd_input_cpu(OpCall& c) {
  const Tensor &grad = c.in[0], &w = c.in[1];
  Tensor& dx = c.out[0];
  const ConvGeom g = conv_geom(dx.shape(), w.shape(), c.i);
  const T* pg = grad.data_as<T>();
  const T* pw = w.data_as<T>();
  T* po = dx.data_as<T>();
  std::memset(po, 0, sizeof(T) * dx.numel());
  for (int64_t n = 0; n < g.N; ++n)
    for (int64_t k = 0; k < g.K; ++k)
      for (int64_t oh = 0; oh < g.OH; ++oh)
        for (int64_t ow = 0; ow < g.OW; ++ow) {
          const T gv = pg[((n * g.K + k) * g.OH + oh) * g.OW + ow];
          for (int64_t ci = 0; ci < g.C; ++ci)
            for (int64_t r = 0; r < g.R; ++r) {
              const int64_t ih = oh * g.sh - g.ph + r;
              if (ih < 0 || ih >= g.H) continue;
              for (int64_t s = 0; s < g.S; ++s) {
                const int64_t iw = ow * g.sw - g.pw + s;
                if (iw < 0 || iw >= g.W) continue;
                po[((n * g.C + ci) * g.H + ih) * g.W + iw] += gv * pw[((k * g.C + ci) * g.R + r) * g.S + s];
              }
            }
        }
}

template <class T>
void conv2d_bwd_weight_cpu(OpCall& c) {
  const Tensor &grad = c.in[0], &x = c.in[1];
  Tensor& dw = c.out[0];
  const ConvGeom g = conv_geom(x.shape(), dw.shape(), c.i);
  const T* pg = grad.data_as<T>();
  const T* px = x.data_as<T>();
  T* po = dw.data_as<T>();
  for (int64_t k = 0; k < g.K; ++k)
    for (int64_t ci = 0; ci < g.C; ++ci)
      for (int64_t r = 0; r < g.R; ++r)
        for (int64_t s = 0; s < g.S; ++s) {
          double acc = 0.0;
          for (int64_t n = 0; n < g.N; ++n)
            for (int64_t oh = 0; oh < g.OH; ++oh) {
              const int64_t ih = oh * g.sh - g.ph + r;
              if (ih < 0 || ih >= g.H) continue;
              for (int64_t ow = 0; ow < g.OW; ++ow) {
                const int64_t iw = ow * g.sw - g.pw + s;
                if (iw < 0 || iw >= g.W) continue;
                acc += static_cast<double>(pg[((n * g.K + k) * g.OH + oh) * g.OW + ow]) *
                       px[((n * g.C + ci) * g.H + ih) * g.W + iw];
              }
            }
          po[((k * g.C + ci) * g.R + r) * g.S + s] = static_cast<T>(acc);
        }
}

template <class T>
void conv2d_bwd_bias_cpu(OpCall& c) {
  const Tensor& grad = c.in[0];
  const int64_t N = grad.shape()[0], K = grad.shape()[1], HW = grad.shape()[2] * grad.shape()[3];
  const T* pg = grad.data_as<T>();
  T* po = c.out[0].data_as<T>();
  for (int64_t k = 0; k < K; ++k) {
    double acc = 0.0;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t i = 0; i < HW; ++i) acc += pg[(n * K + k) * HW + i];
    po[k] = static_cast<T>(acc);
  }
}

// Max pooling ignores NaN whenever the window holds a number; the first maximum wins.
template <class T>
inline int64_t pool_argmax(const T* plane, int64_t H, int64_t W, int64_t oh, int64_t ow, const int64_t* i) {
  const int64_t kh = i[0], kw = i[1], sh = i[2], sw = i[3], ph = i[4], pw = i[5];
  int64_t best = -1;
  T bv = T(0);
  for (int64_t r = 0; r < kh; ++r) {
    const int64_t ih = oh * sh - ph + r;
    if (ih < 0 || ih >= H) continue;
    for (int64_t s = 0; s < kw; ++s) {
      const int64_t iw = ow * sw - pw + s;
      if (iw < 0 || iw >= W) continue;
      const T v = plane[ih * W + iw];
      if (best < 0) { best = ih * W + iw; bv = v; continue; }
      const bool vn = v != v, bn = bv != bv;
      if ((bn && !vn) || (!vn && !bn && v > bv)) { best = ih * W + iw; bv = v; }
    }
  }
  return best;
}

template <class T>
void maxpool_cpu(OpCall& c) {
  const Tensor& x = c.in[0];
  Tensor& out = c.out[0];
  const int64_t NC = x.shape()[0] * x.shape()[1], H = x.shape()[2], W = x.shape()[3];
  const int64_t OH = out.shape()[2], OW = out.shape()[3];
  const T* px = x.data_as<T>();
  T* po = out.data_as<T>();
  for (int64_t p = 0; p < NC; ++p)
    for (int64_t oh = 0; oh < OH; ++oh)
      for (int64_t ow = 0; ow < OW; ++ow) {
        const int64_t a = pool_argmax(px + p * H * W, H, W, oh, ow, c.i);
        po[(p * OH + oh) * OW + ow] = a < 0 ? -std::numeric_limits<T>::infinity() : px[p * H * W + a];
      }
}

template <class T>
void maxpool_bwd_cpu(OpCall& c) {
  const Tensor &x = c.in[0], &g = c.in[1];
  Tensor& dx = c.out[0];
  const int64_t NC = x.shape()[0] * x.shape()[1], H = x.shape()[2], W = x.shape()[3];
  const int64_t OH = g.shape()[2], OW = g.shape()[3];
  const T* px = x.data_as<T>();
  const T* pg = g.data_as<T>();
  T* po = dx.data_as<T>();
  std::memset(po, 0, sizeof(T) * dx.numel());
  for (int64_t p = 0; p < NC; ++p)
    for (int64_t oh = 0; oh < OH; ++oh)
      for (int64_t ow = 0; ow < OW; ++ow) {
        const int64_t a = pool_argmax(px + p * H * W, H, W, oh, ow, c.i);
        if (a >= 0) po[p * H * W + a] += pg[(p * OH + oh) * OW + ow];
      }
}

template <class T>
void layer_norm_cpu(OpCall& c) {
  const Tensor& x = c.in[0];
  const int64_t R = x.shape()[0], D = x.shape()[1];
  const T* px = x.data_as<T>();
  const T* pw = c.in[1].defined() ? c.in[1].data_as<T>() : nullptr;
  const T* pb = c.in[2].defined() ? c.in[2].data_as<T>() : nullptr;
  T* py = c.out[0].data_as<T>();
  float* pm = c.out[1].data_as<float>();
  float* pr = c.out[2].data_as<float>();
  for (int64_t r = 0; r < R; ++r) {
    double m = 0.0, v = 0.0;
    for (int64_t d = 0; d < D; ++d) m += px[r * D + d];
    m /= static_cast<double>(D);
    for (int64_t d = 0; d < D; ++d) { const double z = px[r * D + d] - m; v += z * z; }
    v /= static_cast<double>(D);
    const double rstd = 1.0 / std::sqrt(v + c.f[0]);
    pm[r] = static_cast<float>(m);
    pr[r] = static_cast<float>(rstd);
    for (int64_t d = 0; d < D; ++d) {
      double y = (px[r * D + d] - m) * rstd;
      if (pw) y *= pw[d];
      if (pb) y += pb[d];
      py[r * D + d] = static_cast<T>(y);
    }
  }
}

template <class T>
void layer_norm_bwd_cpu(OpCall& c) {
  const Tensor& x = c.in[0];
  const int64_t R = x.shape()[0], D = x.shape()[1];
  const T* px = x.data_as<T>();
  const T* pw = c.in[1].defined() ? c.in[1].data_as<T>() : nullptr;
  const T* pg = c.in[2].data_as<T>();
  const float* pm = c.in[3].data_as<float>();
  const float* pr = c.in[4].data_as<float>();
  T* pdx = c.out[0].data_as<T>();
  std::vector<double> dw(static_cast<size_t>(D), 0.0), db(static_cast<size_t>(D), 0.0);
  for (int64_t r = 0; r < R; ++r) {
    double s1 = 0.0, s2 = 0.0;
    for (int64_t d = 0; d < D; ++d) {
      const double xh = (px[r * D + d] - pm[r]) * pr[r];
      const double gy = pg[r * D + d] * (pw ? pw[d] : T(1));
      s1 += gy;
      s2 += gy * xh;
      dw[d] += pg[r * D + d] * xh;
      db[d] += pg[r * D + d];
    }
    for (int64_t d = 0; d < D; ++d) {
      const double xh = (px[r * D + d] - pm[r]) * pr[r];
      const double gy = pg[r * D + d] * (pw ? pw[d] : T(1));
      pdx[r * D + d] = static_cast<T>(pr[r] * (gy - s1 / D - xh * s2 / D));
    }
  }
  if (c.out[1].defined()) for (int64_t d = 0; d < D; ++d) c.out[1].data_as<T>()[d] = static_cast<T>(dw[d]);
  if (c.out[2].defined()) for (int64_t d = 0; d < D; ++d) c.out[2].data_as<T>()[d] = static_cast<T>(db[d]);
}

template <class T>
void causal_softmax_cpu(OpCall& c) {
  const Tensor& s = c.in[0];
  const int64_t N = s.shape()[0], Tq = s.shape()[1], Tk = s.shape()[2];
  const T* ps = s.data_as<T>();
  const T* pm = c.in[1].defined() ? c.in[1].data_as<T>() : nullptr;
  T* po = c.out[0].data_as<T>();
  const double scale = c.f[0];
  const bool causal = c.i[0] != 0;
  std::vector<double> row(static_cast<size_t>(Tk));
  for (int64_t n = 0; n < N; ++n)
    for (int64_t i = 0; i < Tq; ++i) {
      double mx = -std::numeric_limits<double>::infinity();
      for (int64_t j = 0; j < Tk; ++j) {
        double v = ps[(n * Tq + i) * Tk + j] * scale;
        if (pm) v += pm[i * Tk + j];
        if (causal && j > i + (Tk - Tq)) v = -std::numeric_limits<double>::infinity();
        row[j] = v;
        mx = std::max(mx, v);
      }
      double sum = 0.0;
      for (int64_t j = 0; j < Tk; ++j) { row[j] = std::exp(row[j] - mx); sum += row[j]; }
      for (int64_t j = 0; j < Tk; ++j) po[(n * Tq + i) * Tk + j] = static_cast<T>(row[j] / sum);
    }
}

template <class T>
void causal_softmax_bwd_cpu(OpCall& c) {
  const Tensor& p = c.in[0];
  const int64_t rows = p.shape()[0] * p.shape()[1], Tk = p.shape()[2];
  const T* pp = p.data_as<T>();
  const T* pg = c.in[1].data_as<T>();
  T* po = c.out[0].data_as<T>();
  const double scale = c.f[0];
  for (int64_t r = 0; r < rows; ++r) {
    double dot = 0.0;
    for (int64_t j = 0; j < Tk; ++j) dot += static_cast<double>(pp[r * Tk + j]) * pg[r * Tk + j];
    for (int64_t j = 0; j < Tk; ++j)
      po[r * Tk + j] = static_cast<T>(pp[r * Tk + j] * (pg[r * Tk + j] - dot) * scale);
  }
}

// p -= lr*wd*p ; m,v moments ; p -= (lr/bc1) * m / (sqrt(v/bc2) + eps)   (eps outside sqrt)
template <class T>
void adam_cpu(OpCall& c) {
  Tensor &p = c.in[0], &m = c.in[1], &v = c.in[2];
  const Tensor& g = c.in[3];
  const double lr = c.f[0], b1 = c.f[1], b2 = c.f[2], eps = c.f[3], wd = c.f[4], bc1 = c.f[5], bc2 = c.f[6],
               gs = c.f[7];
  T* pp = p.data_as<T>();
  T* pm = m.data_as<T>();
  T* pv = v.data_as<T>();
  const size_t gsz = dtype_size(g.dtype());
  const char* pg = static_cast<const char*>(g.data());
  const int64_t n = p.numel();
  for (int64_t i = 0; i < n; ++i) {
    const T gr = static_cast<T>(load_as_double(pg + i * gsz, g.dtype()) * gs);
    pm[i] = pm[i] + static_cast<T>(b1 - 1.0) * pm[i] + static_cast<T>(1.0 - b1) * gr;
    pv[i] = pv[i] + static_cast<T>(b2 - 1.0) * pv[i] + static_cast<T>(1.0 - b2) * (gr * gr);
    const T denom = std::sqrt(pv[i] * static_cast<T>(1.0 / bc2)) + static_cast<T>(eps);
    T w = pp[i];
    if (wd != 0.0) w += static_cast<T>(-lr * wd) * w;
    w += static_cast<T>(-lr / bc1) * (pm[i] / denom);
    pp[i] = w;
  }
  if (c.in[4].defined()) {
    Tensor& model = c.in[4];
    const size_t esz = dtype_size(model.dtype());
    char* pd = static_cast<char*>(model.data());
    for (int64_t i = 0; i < n; ++i) store_from_double(pd + i * esz, model.dtype(), pp[i]);
  }
}

template <class T>
void sgd_cpu(OpCall& c) {
  Tensor& p = c.in[0];
  const Tensor& g = c.in[1];
  const double lr = c.f[0], wd = c.f[1], gs = c.f[2];
  T* pp = p.data_as<T>();
  const size_t gsz = dtype_size(g.dtype());
  const char* pg = static_cast<const char*>(g.data());
  const int64_t n = p.numel();
  for (int64_t i = 0; i < n; ++i) {
    T w = pp[i];
    if (wd != 0.0) w += static_cast<T>(-lr * wd) * w;
    w += static_cast<T>(-lr) * static_cast<T>(load_as_double(pg + i * gsz, g.dtype()) * gs);
    pp[i] = w;
  }
  if (c.in[2].defined()) {
    Tensor& model = c.in[2];
    const size_t esz = dtype_size(model.dtype());
    char* pd = static_cast<char*>(model.data());
    for (int64_t i = 0; i < n; ++i) store_from_double(pd + i * esz, model.dtype(), pp[i]);
  }
}

}  // namespace

void register_cpu_elementwise(KernelRegistry& r);

void register_cpu_kernels(KernelRegistry& r) {
  register_cpu_elementwise(r);
  const uint8_t any = kContiguous | kStrided | kEmpty;
  const uint8_t packed = kContiguous | kEmpty;
#define REG2(OP, FN, NAME, LAY)                                                                     \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CPU, kMaskF32, LAY, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CPU, kMaskF64, LAY, Capability::None}, FN<double>, NAME "_f64");
  REG2(Matmul, matmul_cpu, "cpu_matmul", any) REG2(Linear, linear_cpu, "cpu_linear", any)
  REG2(Softmax, softmax_cpu, "cpu_softmax", packed) REG2(LogSoftmax, log_softmax_cpu, "cpu_log_softmax", packed)
  REG2(SoftmaxBackward, softmax_bwd_cpu, "cpu_softmax_backward", packed)
  REG2(LogSoftmaxBackward, log_softmax_bwd_cpu, "cpu_log_softmax_backward", packed)
  REG2(CrossEntropy, cross_entropy_cpu, "cpu_cross_entropy", packed)
  REG2(CrossEntropyBackward, cross_entropy_bwd_cpu, "cpu_cross_entropy_backward", packed)
  REG2(NllLoss, nll_cpu, "cpu_nll_loss", packed) REG2(NllLossBackward, nll_bwd_cpu, "cpu_nll_loss_backward", packed)
  REG2(Embedding, embedding_cpu, "cpu_embedding", packed)
  REG2(EmbeddingBackward, embedding_bwd_cpu, "cpu_embedding_backward", packed)
  REG2(Conv2d, conv2d_cpu, "cpu_conv2d", packed)
  REG2(Conv2dBackwardInput, conv2d_bwd_input_cpu, "cpu_conv2d_backward_input", packed)
  REG2(Conv2dBackwardWeight, conv2d_bwd_weight_cpu, "cpu_conv2d_backward_weight", packed)
  REG2(Conv2dBackwardBias, conv2d_bwd_bias_cpu, "cpu_conv2d_backward_bias", packed)
  REG2(MaxPool2d, maxpool_cpu, "cpu_maxpool2d", packed) REG2(MaxPool2dBackward, maxpool_bwd_cpu, "cpu_maxpool2d_backward", packed)
  REG2(LayerNorm, layer_norm_cpu, "cpu_layer_norm", packed)
  REG2(LayerNormBackward, layer_norm_bwd_cpu, "cpu_layer_norm_backward", packed)
  REG2(CausalSoftmax, causal_softmax_cpu, "cpu_causal_softmax", packed)
  REG2(CausalSoftmaxBackward, causal_softmax_bwd_cpu, "cpu_causal_softmax_backward", packed)
  REG2(AdamStep, adam_cpu, "cpu_adam_step", packed) REG2(SgdStep, sgd_cpu, "cpu_sgd_step", packed)
#undef REG2
}

}  // namespace ob

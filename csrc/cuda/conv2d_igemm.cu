// conv2d on the tensor cores: the three convolution products are lowered to batched tcgen05
// GEMMs over an unfolded (im2col) copy of the activations.
//
//   fprop   out[n] [K, P]        = W [K, CRS]        @ col[n] [CRS, P]      (+ bias per row)
//   dgrad   dcol[n] [CRS, P]     = W^T [CRS, K]      @ g[n] [K, P]          then fold -> dx
//   wgrad   dW[n] [K, CRS]       = g[n] [K, P]       @ col[n]^T [P, CRS]    then sum over n
//
// with P = OH*OW and CRS = C*R*S padded to a multiple of 8 so that every TMA stride is a
// multiple of 16 bytes.  The weight matrix is shared by all batch entries (batch stride 0),
// transposed operands are MN-major descriptors, nothing is transposed in memory.  Used for
// every floating type when P is a multiple of 8; other cases use the direct kernels.  float32
// products run on whichever GEMM route the float32 matmul precision setting selects (the FMA
// kernel by default).
// ORTHON_CUDA_CONV2D=direct forces the direct kernels.
//
// Replaces (reference project paths): src/backends/cuda/conv2d_cuda.cu:311-2121.
#include <cstdlib>
#include <cstring>

#include <atomic>

#include "ob/cuda_common.cuh"
#include "ob/ops.h"

namespace ob {
namespace cu {

void gemm_launch(const Tensor& A, bool ta, const Tensor& B, bool tb, Tensor& C, const Tensor& bias, bool bias_rows,
                 cudaStream_t st);
void strided_copy_cuda(const Tensor& src, Tensor& dst, cudaStream_t st);

namespace {

constexpr int kThreads = 256;

struct Geom {
  int N, C, H, W, K, R, S, OH, OW, sh, sw, ph, pw, CRS, CRSp, P;
};

Geom make_geom(const Shape& x, const Shape& w, const int64_t* i) {
  Geom g;
  g.N = static_cast<int>(x[0]); g.C = static_cast<int>(x[1]); g.H = static_cast<int>(x[2]); g.W = static_cast<int>(x[3]);
  g.K = static_cast<int>(w[0]); g.R = static_cast<int>(w[2]); g.S = static_cast<int>(w[3]);
  g.sh = static_cast<int>(i[0]); g.sw = static_cast<int>(i[1]); g.ph = static_cast<int>(i[2]); g.pw = static_cast<int>(i[3]);
  g.OH = (g.H + 2 * g.ph - g.R) / g.sh + 1;
  g.OW = (g.W + 2 * g.pw - g.S) / g.sw + 1;
  g.CRS = g.C * g.R * g.S;
  g.CRSp = (g.CRS + 7) & ~7;
  g.P = g.OH * g.OW;
  return g;
}

// col[n][crs][p] = x[n][c][oh*sh-ph+r][ow*sw-pw+s]  (0 outside the image and in padded rows).
// One block per (n, crs) row of the column matrix: the filter tap is decoded once per block, every
// thread produces one 16-byte pack of consecutive output positions (8 for 16-bit types, 4 for
// float32) with 32-bit index arithmetic (P is a multiple of 8 on this path).
template <class T>
__global__ void unfold_kernel(const T* __restrict__ x, T* __restrict__ col, Geom g) {
  const int crs = blockIdx.x, n = blockIdx.y;
  T* out = col + (static_cast<int64_t>(n) * g.CRSp + crs) * g.P;
  const bool live = crs < g.CRS;
  const int s = crs % g.S, r = (crs / g.S) % g.R, c = crs / (g.S * g.R);
  const T* img = x + (static_cast<int64_t>(n) * g.C + (live ? c : 0)) * g.H * g.W;
  constexpr int N = Pack<T>::N;
  for (int v = threadIdx.x; v < g.P / N; v += blockDim.x) {
    Pack<T> pk;
    int oh = (v * N) / g.OW, ow = (v * N) - oh * g.OW;
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const int ih = oh * g.sh - g.ph + r, iw = ow * g.sw - g.pw + s;
      pk.v[e] = (live && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? img[ih * g.W + iw] : from_f<T>(0.f);
      if (++ow == g.OW) { ow = 0; ++oh; }
    }
    store_pack(out + v * N, pk);
  }
}

// dx[n][c][ih][iw] = sum over (r, s) of dcol[n][(c,r,s)][oh*OW+ow] where the window maps back.
// grid = (ceil(H*W / 256), C, N): channel and image come from the block index, so the per-pixel
// work is 32-bit arithmetic only.
template <class T>
__global__ void fold_kernel(const T* __restrict__ dcol, T* __restrict__ dx, Geom g) {
  const int c = blockIdx.y, n = blockIdx.z;
  const int pix = blockIdx.x * blockDim.x + threadIdx.x;
  if (pix >= g.H * g.W) return;
  const int ih = pix / g.W, iw = pix - ih * g.W;
  const T* rows = dcol + (static_cast<int64_t>(n) * g.CRSp + static_cast<int64_t>(c) * g.R * g.S) * g.P;
  float acc = 0.f;
  for (int r = 0; r < g.R; ++r) {
    const int th = ih + g.ph - r;
    if (th < 0 || th % g.sh != 0 || th / g.sh >= g.OH) continue;
    for (int s = 0; s < g.S; ++s) {
      const int tw = iw + g.pw - s;
      if (tw < 0 || tw % g.sw != 0 || tw / g.sw >= g.OW) continue;
      acc += to_f(rows[static_cast<int64_t>(r * g.S + s) * g.P + (th / g.sh) * g.OW + tw / g.sw]);
    }
  }
  dx[(static_cast<int64_t>(n) * g.C + c) * g.H * g.W + pix] = from_f<T>(acc);
}

// wp[k][crs] = w[k][crs] for crs < CRS else 0
template <class T>
__global__ void pad_weight_kernel(const T* __restrict__ w, T* __restrict__ wp, int K, int CRS, int CRSp) {
  const int64_t total = static_cast<int64_t>(K) * CRSp;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int crs = static_cast<int>(i % CRSp), k = static_cast<int>(i / CRSp);
    wp[i] = crs < CRS ? w[static_cast<int64_t>(k) * CRS + crs] : from_f<T>(0.f);
  }
}

template <class T>
Tensor padded_weight(const Tensor& w, const Geom& g, cudaStream_t st) {
  Tensor wp = Tensor::empty({g.K, g.CRSp}, w.dtype(), w.device());
  if (g.CRSp == g.CRS) {
    OB_CUDA(cudaMemcpyAsync(wp.data(), w.data(), wp.nbytes(), cudaMemcpyDeviceToDevice, st));
  } else {
    pad_weight_kernel<T><<<ew_grid(wp.numel(), kThreads, sm_count_for(w)), kThreads, 0, st>>>(w.data_as<T>(), wp.data_as<T>(), g.K, g.CRS, g.CRSp);
  }
  return wp;
}

template <class T>
Tensor unfold(const Tensor& x, const Geom& g, cudaStream_t st) {
  Tensor col = Tensor::empty({g.N, g.CRSp, g.P}, x.dtype(), x.device());
  unfold_kernel<T><<<dim3(static_cast<unsigned>(g.CRSp), static_cast<unsigned>(g.N)), 128, 0, st>>>(x.data_as<T>(), col.data_as<T>(), g);
  return col;
}

Tensor broadcast_batch(const Tensor& m2d, int64_t n) {  // [rows, cols] -> [n, rows, cols] with batch stride 0
  return Tensor::view_of(m2d, Layout(Shape{n, m2d.shape()[0], m2d.shape()[1]}, Shape{0, m2d.strides()[0], m2d.strides()[1]}, m2d.offset()));
}

}  // namespace

std::atomic<int> g_conv_force{0};  // 0 = planner, 1 = direct kernels, 2 = tcgen05 lowering required
std::atomic<int> g_conv_last{0};   // 1 = direct, 2 = tcgen05 lowering
void set_conv_route(int route) { g_conv_force.store(route, std::memory_order_relaxed); }
int last_conv_route() { return g_conv_last.load(std::memory_order_relaxed); }
void note_conv_route(int route) { g_conv_last.store(route, std::memory_order_relaxed); }
int conv_forced_route() { return g_conv_force.load(std::memory_order_relaxed); }

bool conv_igemm_enabled(const Tensor& x, const Geom* unused = nullptr) {
  (void)unused;
  if (g_conv_force.load(std::memory_order_relaxed) == 1) return false;
  const char* env = std::getenv("ORTHON_CUDA_CONV2D");
  if (env && std::strcmp(env, "direct") == 0) return false;
  if (x.dtype() != DType::BF16 && x.dtype() != DType::F16 && x.dtype() != DType::F32) return false;
  return Runtime::instance().cuda(x.device().index).supports_tcgen05();
}

template <class T>
bool conv_fprop_igemm(OpCall& c) {
  const Tensor &x = c.in[0], &w = c.in[1];
  if (!conv_igemm_enabled(x)) return false;
  const Geom g = make_geom(x.shape(), w.shape(), c.i);
  if (g.P % 8 != 0) return false;
  cudaStream_t st = stream_of(c);
  Tensor wp = padded_weight<T>(w, g, st);
  Tensor col = unfold<T>(x, g, st);
  Tensor out3 = Tensor::view_of(c.out[0], Layout(Shape{g.N, g.K, g.P}));
  gemm_launch(broadcast_batch(wp, g.N), false, col, false, out3, c.in[2], true, st);
  check_launch("conv2d (tcgen05)");
  return true;
}

template <class T>
bool conv_dgrad_igemm(OpCall& c) {
  const Tensor &gy = c.in[0], &w = c.in[1];
  Tensor& dx = c.out[0];
  if (!conv_igemm_enabled(gy)) return false;
  const Geom g = make_geom(dx.shape(), w.shape(), c.i);
  if (g.P % 8 != 0) return false;
  cudaStream_t st = stream_of(c);
  Tensor wp = padded_weight<T>(w, g, st);
  Tensor g3 = Tensor::view_of(gy, Layout(Shape{g.N, g.K, g.P}, Layout::contiguous_strides({g.N, g.K, g.P}), gy.offset()));
  Tensor dcol = Tensor::empty({g.N, g.CRSp, g.P}, gy.dtype(), gy.device());
  gemm_launch(broadcast_batch(wp, g.N), true, g3, false, dcol, Tensor(), false, st);
  fold_kernel<T><<<dim3(static_cast<unsigned>((g.H * g.W + kThreads - 1) / kThreads), static_cast<unsigned>(g.C), static_cast<unsigned>(g.N)), kThreads, 0, st>>>(
      dcol.data_as<T>(), dx.data_as<T>(), g);
  check_launch("conv2d dgrad (tcgen05)");
  return true;
}

template <class T>
bool conv_wgrad_igemm(OpCall& c) {
  const Tensor &gy = c.in[0], &x = c.in[1];
  Tensor& dw = c.out[0];
  if (!conv_igemm_enabled(gy)) return false;
  const Geom g = make_geom(x.shape(), dw.shape(), c.i);
  if (g.P % 8 != 0) return false;
  cudaStream_t st = stream_of(c);
  Tensor col = unfold<T>(x, g, st);
  Tensor g3 = Tensor::view_of(gy, Layout(Shape{g.N, g.K, g.P}, Layout::contiguous_strides({g.N, g.K, g.P}), gy.offset()));
  Tensor per_image = Tensor::empty({g.N, g.K, g.CRSp}, gy.dtype(), gy.device());
  gemm_launch(g3, false, col, true, per_image, Tensor(), false, st);
  Tensor dwp = Tensor::empty({g.K, g.CRSp}, gy.dtype(), gy.device());
  OpCall s;
  s.in[0] = per_image;
  s.out[0] = dwp;
  s.i[0] = 1; s.i[1] = g.N; s.i[2] = static_cast<int64_t>(g.K) * g.CRSp;
  s.stream = c.stream;
  default_dispatcher().run(DispatchRequest{OperatorId::Sum, gy.device(), gy.dtype(), kContiguous}, s);
  Tensor src = Tensor::view_of(dwp, Layout(Shape{g.K, g.CRS}, Shape{g.CRSp, 1}, 0));
  Tensor dst = Tensor::view_of(dw, Layout(Shape{g.K, g.CRS}));
  strided_copy_cuda(src, dst, st);
  check_launch("conv2d wgrad (tcgen05)");
  return true;
}

template bool conv_fprop_igemm<__nv_bfloat16>(OpCall&);
template bool conv_fprop_igemm<__half>(OpCall&);
template bool conv_dgrad_igemm<__nv_bfloat16>(OpCall&);
template bool conv_dgrad_igemm<__half>(OpCall&);
template bool conv_wgrad_igemm<__nv_bfloat16>(OpCall&);
template bool conv_wgrad_igemm<__half>(OpCall&);
template bool conv_fprop_igemm<float>(OpCall&);
template bool conv_dgrad_igemm<float>(OpCall&);
template bool conv_wgrad_igemm<float>(OpCall&);

}  // namespace cu
}  // namespace ob

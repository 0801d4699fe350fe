// conv2d (NCHW / OIHW) forward, input gradient, weight gradient and bias gradient.
//
// Direct kernels with float32 accumulation for float32 / float16 / bfloat16 tensors.  The
// weight and bias gradients are deterministic block reductions (one block per weight
// element / output channel), never atomics.
//
// Replaces (reference project paths): src/backends/cuda/conv2d_cuda.cu:102-2185.
#include "ob/cuda_common.cuh"

namespace ob {
namespace cu {

template <class T> bool conv_fprop_igemm(OpCall& c);
template <class T> bool conv_dgrad_igemm(OpCall& c);
template <class T> bool conv_wgrad_igemm(OpCall& c);
// Implicit GEMM (gather in the producer, no column matrix): 16-bit types only.
template <class T> bool conv_fprop_tc05(OpCall& c);
template <class T> bool conv_dgrad_tc05(OpCall& c);
template <class T> bool conv_wgrad_tc05(OpCall& c);
template <> inline bool conv_fprop_tc05<float>(OpCall&) { return false; }
template <> inline bool conv_dgrad_tc05<float>(OpCall&) { return false; }
template <> inline bool conv_wgrad_tc05<float>(OpCall&) { return false; }
void note_conv_route(int route);  // diagnostics: 1 = direct kernels, 2 = tcgen05 lowering, 3 = tcgen05 implicit GEMM
int conv_forced_route();

namespace {

constexpr int kThreads = 256;

struct ConvGeom {
  int N, C, H, W, K, R, S, OH, OW, sh, sw, ph, pw;
};

ConvGeom geom_of(const Shape& x, const Shape& w, const int64_t* i) {
  ConvGeom g;
  g.N = static_cast<int>(x[0]); g.C = static_cast<int>(x[1]); g.H = static_cast<int>(x[2]); g.W = static_cast<int>(x[3]);
  g.K = static_cast<int>(w[0]); g.R = static_cast<int>(w[2]); g.S = static_cast<int>(w[3]);
  g.sh = static_cast<int>(i[0]); g.sw = static_cast<int>(i[1]); g.ph = static_cast<int>(i[2]); g.pw = static_cast<int>(i[3]);
  g.OH = (g.H + 2 * g.ph - g.R) / g.sh + 1;
  g.OW = (g.W + 2 * g.pw - g.S) / g.sw + 1;
  return g;
}

template <class T>
__global__ void conv_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                T* __restrict__ y, ConvGeom g) {
  const int64_t n_out = static_cast<int64_t>(g.N) * g.K * g.OH * g.OW;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_out; i += stride) {
    const int ow = static_cast<int>(i % g.OW), oh = static_cast<int>((i / g.OW) % g.OH);
    const int k = static_cast<int>((i / (static_cast<int64_t>(g.OW) * g.OH)) % g.K);
    const int n = static_cast<int>(i / (static_cast<int64_t>(g.OW) * g.OH * g.K));
    float acc = b ? to_f(b[k]) : 0.f;
    for (int c = 0; c < g.C; ++c) {
      const T* xp = x + (static_cast<int64_t>(n) * g.C + c) * g.H * g.W;
      const T* wp = w + (static_cast<int64_t>(k) * g.C + c) * g.R * g.S;
      for (int r = 0; r < g.R; ++r) {
        const int ih = oh * g.sh - g.ph + r;
        if (ih < 0 || ih >= g.H) continue;
        for (int s = 0; s < g.S; ++s) {
          const int iw = ow * g.sw - g.pw + s;
          if (iw < 0 || iw >= g.W) continue;
          acc = fmaf(to_f(xp[ih * g.W + iw]), to_f(wp[r * g.S + s]), acc);
        }
      }
    }
    y[i] = from_f<T>(acc);
  }
}

// dx[n,c,ih,iw] = sum_{k,r,s : (ih+ph-r) % sh == 0 ...} g[n,k,oh,ow] * w[k,c,r,s]
template <class T>
__global__ void conv_dgrad_kernel(const T* __restrict__ gy, const T* __restrict__ w, T* __restrict__ dx, ConvGeom g) {
  const int64_t n_in = static_cast<int64_t>(g.N) * g.C * g.H * g.W;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_in; i += stride) {
    const int iw = static_cast<int>(i % g.W), ih = static_cast<int>((i / g.W) % g.H);
    const int c = static_cast<int>((i / (static_cast<int64_t>(g.W) * g.H)) % g.C);
    const int n = static_cast<int>(i / (static_cast<int64_t>(g.W) * g.H * g.C));
    float acc = 0.f;
    for (int r = 0; r < g.R; ++r) {
      const int th = ih + g.ph - r;
      if (th < 0 || th % g.sh != 0) continue;
      const int oh = th / g.sh;
      if (oh >= g.OH) continue;
      for (int s = 0; s < g.S; ++s) {
        const int tw = iw + g.pw - s;
        if (tw < 0 || tw % g.sw != 0) continue;
        const int ow = tw / g.sw;
        if (ow >= g.OW) continue;
        for (int k = 0; k < g.K; ++k)
          acc = fmaf(to_f(gy[((static_cast<int64_t>(n) * g.K + k) * g.OH + oh) * g.OW + ow]),
                     to_f(w[((static_cast<int64_t>(k) * g.C + c) * g.R + r) * g.S + s]), acc);
      }
    }
    dx[i] = from_f<T>(acc);
  }
}

// One block per weight element; threads stride over (n, oh, ow).
template <class T>
__global__ void conv_wgrad_kernel(const T* __restrict__ gy, const T* __restrict__ x, T* __restrict__ dw, ConvGeom g) {
  __shared__ float smem[32];
  const int64_t widx = blockIdx.x;
  const int s = static_cast<int>(widx % g.S), r = static_cast<int>((widx / g.S) % g.R);
  const int c = static_cast<int>((widx / (g.S * g.R)) % g.C), k = static_cast<int>(widx / (static_cast<int64_t>(g.S) * g.R * g.C));
  const int64_t total = static_cast<int64_t>(g.N) * g.OH * g.OW;
  float acc = 0.f;
  for (int64_t j = threadIdx.x; j < total; j += blockDim.x) {
    const int ow = static_cast<int>(j % g.OW), oh = static_cast<int>((j / g.OW) % g.OH);
    const int n = static_cast<int>(j / (static_cast<int64_t>(g.OW) * g.OH));
    const int ih = oh * g.sh - g.ph + r, iw = ow * g.sw - g.pw + s;
    if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) continue;
    acc = fmaf(to_f(gy[((static_cast<int64_t>(n) * g.K + k) * g.OH + oh) * g.OW + ow]),
               to_f(x[((static_cast<int64_t>(n) * g.C + c) * g.H + ih) * g.W + iw]), acc);
  }
  acc = block_sum(acc, smem);
  if (threadIdx.x == 0) dw[widx] = from_f<T>(acc);
}

template <class T>
__global__ void conv_bgrad_kernel(const T* __restrict__ gy, T* __restrict__ db, int N, int K, int64_t HW) {
  __shared__ float smem[32];
  const int k = blockIdx.x;
  float acc = 0.f;
  const int64_t total = static_cast<int64_t>(N) * HW;
  for (int64_t j = threadIdx.x; j < total; j += blockDim.x) {
    const int64_t n = j / HW, i = j - n * HW;
    acc += to_f(gy[(n * K + k) * HW + i]);
  }
  acc = block_sum(acc, smem);
  if (threadIdx.x == 0) db[k] = from_f<T>(acc);
}

template <class T>
void k_conv(OpCall& c) {
  if (conv_forced_route() == 0 && conv_fprop_tc05<T>(c)) { note_conv_route(3); return; }
  if (conv_fprop_igemm<T>(c)) { note_conv_route(2); return; }
  note_conv_route(1);
  const ConvGeom g = geom_of(c.in[0].shape(), c.in[1].shape(), c.i);
  conv_fwd_kernel<T><<<ew_grid(c.out[0].numel(), kThreads, sm_count_for(c.in[0])), kThreads, 0, stream_of(c)>>>(
      c.in[0].data_as<T>(), c.in[1].data_as<T>(), c.in[2].defined() ? c.in[2].data_as<T>() : nullptr, c.out[0].data_as<T>(), g);
  check_launch("conv2d");
}

template <class T>
void k_conv_dgrad(OpCall& c) {
  if (conv_forced_route() == 0 && conv_dgrad_tc05<T>(c)) { note_conv_route(3); return; }
  if (conv_dgrad_igemm<T>(c)) { note_conv_route(2); return; }
  note_conv_route(1);
  const ConvGeom g = geom_of(c.out[0].shape(), c.in[1].shape(), c.i);
  conv_dgrad_kernel<T><<<ew_grid(c.out[0].numel(), kThreads, sm_count_for(c.in[0])), kThreads, 0, stream_of(c)>>>(
      c.in[0].data_as<T>(), c.in[1].data_as<T>(), c.out[0].data_as<T>(), g);
  check_launch("conv2d backward input");
}

template <class T>
void k_conv_wgrad(OpCall& c) {
  if (conv_forced_route() == 0 && conv_wgrad_tc05<T>(c)) { note_conv_route(3); return; }
  if (conv_wgrad_igemm<T>(c)) { note_conv_route(2); return; }
  note_conv_route(1);
  const ConvGeom g = geom_of(c.in[1].shape(), c.out[0].shape(), c.i);
  conv_wgrad_kernel<T><<<static_cast<unsigned>(c.out[0].numel()), kThreads, 0, stream_of(c)>>>(
      c.in[0].data_as<T>(), c.in[1].data_as<T>(), c.out[0].data_as<T>(), g);
  check_launch("conv2d backward weight");
}

template <class T>
void k_conv_bgrad(OpCall& c) {
  const Tensor& gy = c.in[0];
  conv_bgrad_kernel<T><<<static_cast<unsigned>(gy.shape()[1]), kThreads, 0, stream_of(c)>>>(
      gy.data_as<T>(), c.out[0].data_as<T>(), static_cast<int>(gy.shape()[0]), static_cast<int>(gy.shape()[1]),
      gy.shape()[2] * gy.shape()[3]);
  check_launch("conv2d backward bias");
}

}  // namespace

void register_cuda_conv(KernelRegistry& r) {
  const uint8_t packed = kContiguous | kEmpty;
#define REG3(OP, FN, NAME)                                                                                      \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, kMaskF32, packed, Capability::None}, FN<float>, NAME "_f32"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::F16), packed, Capability::None}, FN<__half>, NAME "_f16"); \
  r.add_kernel(OperatorId::OP, Constraints{Backend::CUDA, dtype_bit(DType::BF16), packed, Capability::Bf16}, FN<__nv_bfloat16>, NAME "_bf16");
  REG3(Conv2d, k_conv, "sm100_conv2d_direct") REG3(Conv2dBackwardInput, k_conv_dgrad, "sm100_conv2d_dgrad")
  REG3(Conv2dBackwardWeight, k_conv_wgrad, "sm100_conv2d_wgrad") REG3(Conv2dBackwardBias, k_conv_bgrad, "sm100_conv2d_bgrad")
#undef REG3
}

}  // namespace cu
}  // namespace ob

// Host<->device and device<->device transfers behind the `to` operator, pinned host
// memory, and the aggregate CUDA kernel registration.
//
// Parity (reference project paths): src/backends/cuda/adapters.cpp:25-62,
// src/runtime/cuda_context.cpp:203-278 (h2d snapshot, blocking d2h, peer copy).
#include <cuda_runtime_api.h>

#include "ob/kernels.h"
#include "ob/ops.h"

namespace ob {
namespace cu {

void strided_copy_cuda(const Tensor& src, Tensor& dst, cudaStream_t st);
void register_cuda_elementwise(KernelRegistry& r);
void register_cuda_reduce(KernelRegistry& r);
void register_cuda_nn(KernelRegistry& r);
void register_cuda_gemm(KernelRegistry& r);
void register_cuda_conv(KernelRegistry& r);

namespace {

void to_cuda_kernel(OpCall& c) {
  const Tensor& src = c.in[0];
  Tensor& dst = c.out[0];
  if (src.device().is_cpu()) {
    // Host -> device: pack on the host when strided, then one async copy.  Pageable
    // sources are synchronized so the caller may reuse the host memory immediately.
    Tensor packed = src.is_contiguous() ? src : ops::clone(src);
    DeviceGuard g(dst.device().index);
    cudaStream_t st = static_cast<cudaStream_t>(Runtime::instance().stream_for(dst.device()));
    OB_CUDA(cudaMemcpyAsync(dst.data(), packed.data(), dst.nbytes(), cudaMemcpyHostToDevice, st));
    if (c.i[0] == 0) OB_CUDA(cudaStreamSynchronize(st));
    return;
  }
  DeviceGuard g(src.device().index);
  cudaStream_t st = static_cast<cudaStream_t>(Runtime::instance().stream_for(src.device()));
  if (dst.device().is_cpu()) {
    Tensor packed = src;
    if (!src.is_contiguous()) {
      packed = Tensor::empty(src.shape(), src.dtype(), src.device());
      strided_copy_cuda(src, packed, st);
    }
    OB_CUDA(cudaMemcpyAsync(dst.data(), packed.data(), dst.nbytes(), cudaMemcpyDeviceToHost, st));
    OB_CUDA(cudaStreamSynchronize(st));
    return;
  }
  if (dst.device() == src.device()) {
    strided_copy_cuda(src, dst, st);
    return;
  }
  // Peer copy: pack on the source device, order both compute streams around the copy.
  Tensor packed = src;
  if (!src.is_contiguous()) {
    packed = Tensor::empty(src.shape(), src.dtype(), src.device());
    strided_copy_cuda(src, packed, st);
  }
  OB_CUDA(cudaStreamSynchronize(st));
  cudaStream_t dst_st = static_cast<cudaStream_t>(Runtime::instance().stream_for(dst.device()));
  OB_CUDA(cudaMemcpyPeerAsync(dst.data(), dst.device().index, packed.data(), src.device().index, dst.nbytes(), dst_st));
  OB_CUDA(cudaStreamSynchronize(dst_st));
}

void to_cpu_kernel(OpCall& c) {
  OpCall d;
  d.in[0] = c.in[0];
  d.out[0] = c.out[0];
  const Tensor& src = c.in[0];
  const bool strided = !src.is_contiguous();
  default_dispatcher().run(DispatchRequest{OperatorId::Contiguous, Device(), src.dtype(),
                                           static_cast<uint8_t>(strided ? kStrided : kContiguous)}, d);
}

}  // namespace

// Page-locked host tensor; transfers from it can be truly asynchronous.
Tensor pinned_empty(const Shape& shape, DType dtype) {
  const size_t bytes = static_cast<size_t>(Layout::checked_numel(shape)) * dtype_size(dtype);
  void* p = nullptr;
  OB_CUDA(cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault));
  auto buf = std::make_shared<Buffer>(Allocation::external(p, bytes, Device(), [p] { cudaFreeHost(p); }));
  return Tensor(std::make_shared<TensorImpl>(buf, Layout(shape), dtype));
}

// Async host->device copy into an existing device tensor on the given stream kind
// (0 = compute, 1 = copy).  The source must stay alive and unchanged until the copy ran.
void copy_h2d_async(Tensor& dst, const Tensor& src, int stream_kind) {
  if (!dst.device().is_cuda() || !src.device().is_cpu()) throw std::invalid_argument("copy_h2d_async: expects host -> device");
  if (!dst.is_contiguous() || !src.is_contiguous() || dst.nbytes() != src.nbytes() || dst.dtype() != src.dtype())
    throw std::invalid_argument("copy_h2d_async: tensors must be contiguous with identical dtype and size");
  CudaContext& ctx = Runtime::instance().cuda(dst.device().index);
  DeviceGuard g(ctx.device());
  cudaStream_t st = static_cast<cudaStream_t>(stream_kind == 1 ? ctx.copy_stream() : ctx.current_stream());
  OB_CUDA(cudaMemcpyAsync(dst.data(), src.data(), dst.nbytes(), cudaMemcpyHostToDevice, st));
  if (stream_kind == 1) dst.impl()->buffer()->allocation().record_stream(ctx.copy_stream());
  dst.bump_version();
}

void copy_d2h_async(Tensor& dst, const Tensor& src) {
  if (!src.device().is_cuda() || !dst.device().is_cpu()) throw std::invalid_argument("copy_d2h_async: expects device -> host");
  if (!dst.is_contiguous() || !src.is_contiguous() || dst.nbytes() != src.nbytes() || dst.dtype() != src.dtype())
    throw std::invalid_argument("copy_d2h_async: tensors must be contiguous with identical dtype and size");
  CudaContext& ctx = Runtime::instance().cuda(src.device().index);
  DeviceGuard g(ctx.device());
  OB_CUDA(cudaMemcpyAsync(dst.data(), src.data(), dst.nbytes(), cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(ctx.current_stream())));
  dst.bump_version();
}

}  // namespace cu

void register_cuda_kernels(KernelRegistry& r) {
  const uint8_t any = kContiguous | kStrided | kEmpty;
  r.add_kernel(OperatorId::To, Constraints{Backend::CUDA, kMaskAll, any, Capability::None}, cu::to_cuda_kernel, "cuda_transfer");
  r.add_kernel(OperatorId::To, Constraints{Backend::CPU, kMaskAll, any, Capability::None}, cu::to_cpu_kernel, "cpu_copy");
  cu::register_cuda_elementwise(r);
  cu::register_cuda_reduce(r);
  cu::register_cuda_nn(r);
  cu::register_cuda_gemm(r);
  cu::register_cuda_conv(r);
}

}  // namespace ob

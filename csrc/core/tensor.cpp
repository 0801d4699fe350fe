// Buffer / TensorImpl / Tensor.
#include "ob/tensor.h"

#include "ob/ops.h"

namespace ob {

Buffer::Buffer(Device dev, size_t bytes)
    : alloc_(MemoryPool::instance().acquire(dev, bytes, Runtime::instance().stream_for(dev))) {}

TensorImpl::TensorImpl(const Shape& shape, DType dtype, Device dev) : layout_(shape), dtype_(dtype) {
  const size_t esz = dtype_size(dtype);
  const int64_t n = layout_.numel();
  if (n != 0 && static_cast<uint64_t>(n) > (~size_t(0)) / esz)
    throw std::overflow_error("tensor byte size overflows size_t");
  buf_ = std::make_shared<Buffer>(dev, static_cast<size_t>(n) * esz);
}

TensorImpl::TensorImpl(std::shared_ptr<Buffer> buf, Layout layout, DType dtype)
    : buf_(std::move(buf)), layout_(std::move(layout)), dtype_(dtype) {
  layout_.validate_bounds(buf_->bytes(), dtype_size(dtype_));
}

void* TensorImpl::data() const {
  if (layout_.numel() == 0 || buf_->data() == nullptr) return nullptr;
  return static_cast<char*>(buf_->data()) + layout_.offset() * static_cast<int64_t>(dtype_size(dtype_));
}

void TensorImpl::rebind(const TensorImpl& other) {
  buf_ = other.buf_;
  layout_ = other.layout_;
  dtype_ = other.dtype_;
}

Tensor Tensor::empty(const Shape& shape, DType dtype, Device dev) {
  return Tensor(std::make_shared<TensorImpl>(shape, dtype, dev));
}

Tensor Tensor::zeros(const Shape& shape, DType dtype, Device dev) {
  Tensor t = empty(shape, dtype, dev);
  ops::fill_raw(t, 0.0);
  return t;
}

Tensor Tensor::full(const Shape& shape, double value, DType dtype, Device dev) {
  Tensor t = empty(shape, dtype, dev);
  ops::fill_raw(t, value);
  return t;
}

Tensor Tensor::scalar(double value, DType dtype, Device dev) { return full({1}, value, dtype, dev); }

Tensor Tensor::view_of(const Tensor& base, Layout layout) {
  return Tensor(std::make_shared<TensorImpl>(base.impl()->buffer(), std::move(layout), base.dtype()));
}

Tensor Tensor::view_of(const Tensor& base, Layout layout, DType dtype) {
  return Tensor(std::make_shared<TensorImpl>(base.impl()->buffer(), std::move(layout), dtype));
}

int64_t Tensor::size(int d) const {
  const int n = ndim();
  if (d < 0) d += n;
  OB_CHECK_ARG(d >= 0 && d < n, "dimension out of range");
  return shape()[d];
}

int64_t Tensor::stride(int d) const {
  const int n = ndim();
  if (d < 0) d += n;
  OB_CHECK_ARG(d >= 0 && d < n, "dimension out of range");
  return strides()[d];
}

Tensor& Tensor::requires_grad_(bool on) {
  if (on && !dtype_is_floating(dtype()))
    throw std::invalid_argument("only floating point tensors can require gradients");
  if (!is_leaf() && !on)
    throw std::invalid_argument("requires_grad can only be cleared on leaf tensors");
  impl_->ag().requires_grad = on;
  return *this;
}

void Tensor::set_grad(const Tensor& g) {
  if (!g.defined()) {
    impl_->ag().grad.reset();
    return;
  }
  if (g.shape() != shape()) throw std::invalid_argument("set_grad: gradient shape must match the tensor");
  if (g.dtype() != dtype()) throw std::invalid_argument("set_grad: gradient dtype must match the tensor");
  if (g.device() != device()) throw std::invalid_argument("set_grad: gradient device must match the tensor");
  impl_->ag().grad = g.detach().impl();
}

void Tensor::zero_grad() { impl_->ag().grad.reset(); }

void Tensor::backward(bool retain_graph) const { AutogradEngine::backward(*this, retain_graph); }

Tensor Tensor::detach() const {
  if (!impl_->ag().requires_grad && !impl_->ag().grad_fn) return *this;
  return Tensor(std::make_shared<TensorImpl>(impl_->buffer(), impl_->layout(), impl_->dtype()));
}

}  // namespace ob

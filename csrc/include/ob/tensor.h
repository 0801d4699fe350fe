// Buffer, TensorImpl, Tensor and the autograd graph types.
//
// A Buffer is the shared physical identity of every alias of one allocation and
// carries the mutation generation that saved-tensor checks compare.  A TensorImpl
// is one logical tensor: Buffer + Layout + dtype + per-identity autograd metadata.
// Tensor is the cheap value handle.
//
// Parity (reference project paths): include/orthon/core/{buffer,tensor_impl,tensor,
// autograd_meta}.h, include/orthon/autograd/{node,engine,grad_mode}.h,
// src/autograd/{engine,node,grad_mode}.cpp.
#pragma once
#include <atomic>
#include <functional>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "ob/core.h"
#include "ob/runtime.h"

namespace ob {

class Node;
class TensorImpl;
class Tensor;

class Buffer {
 public:
  Buffer(Device dev, size_t bytes);
  explicit Buffer(Allocation a) : alloc_(std::move(a)) {}
  void* data() const { return alloc_.data(); }
  size_t bytes() const { return alloc_.bytes(); }
  size_t capacity() const { return alloc_.capacity(); }
  Device device() const { return alloc_.device(); }
  uint64_t version() const { return version_.load(std::memory_order_acquire); }
  void bump_version() { version_.fetch_add(1, std::memory_order_acq_rel); }
  Allocation& allocation() { return alloc_; }

 private:
  Allocation alloc_;
  std::atomic<uint64_t> version_{0};
};

enum class History : uint8_t { None, Live, Released };

struct AutogradMeta {
  bool requires_grad = false;
  std::shared_ptr<TensorImpl> grad;
  std::shared_ptr<Node> grad_fn;
  History history = History::None;
  std::vector<std::function<void()>> post_accumulate_hooks;
  std::vector<std::pair<uint64_t, std::function<void()>>> finalizers;
  // Optional preassigned gradient storage (a view into a reducer bucket).  When set,
  // leaf gradients are written into it and `.grad` aliases it.
  std::shared_ptr<TensorImpl> grad_slot;
};

class TensorImpl {
 public:
  TensorImpl(const Shape& shape, DType dtype, Device dev);                         // allocating
  TensorImpl(std::shared_ptr<Buffer> buf, Layout layout, DType dtype);              // view
  const std::shared_ptr<Buffer>& buffer() const { return buf_; }
  const Layout& layout() const { return layout_; }
  DType dtype() const { return dtype_; }
  Device device() const { return buf_->device(); }
  void* data() const;  // base + offset; nullptr for empty tensors
  AutogradMeta& ag() { return ag_; }
  const AutogradMeta& ag() const { return ag_; }
  // Replaces storage, layout and dtype while keeping this identity (Module transforms).
  void rebind(const TensorImpl& other);

 private:
  std::shared_ptr<Buffer> buf_;
  Layout layout_;
  DType dtype_;
  AutogradMeta ag_;
};

class Tensor {
 public:
  Tensor() = default;
  explicit Tensor(std::shared_ptr<TensorImpl> impl) : impl_(std::move(impl)) {}
  static Tensor empty(const Shape& shape, DType dtype, Device dev);
  static Tensor zeros(const Shape& shape, DType dtype, Device dev);
  static Tensor full(const Shape& shape, double value, DType dtype, Device dev);
  static Tensor scalar(double value, DType dtype, Device dev);  // rank-1 [1]
  static Tensor view_of(const Tensor& base, Layout layout);
  static Tensor view_of(const Tensor& base, Layout layout, DType dtype);

  bool defined() const { return static_cast<bool>(impl_); }
  const std::shared_ptr<TensorImpl>& impl() const { return impl_; }
  TensorImpl* raw() const { return impl_.get(); }
  const Shape& shape() const { return impl_->layout().shape(); }
  const Shape& strides() const { return impl_->layout().strides(); }
  int64_t size(int d) const;
  int64_t stride(int d) const;
  int64_t numel() const { return impl_->layout().numel(); }
  int ndim() const { return impl_->layout().ndim(); }
  int64_t offset() const { return impl_->layout().offset(); }
  bool is_contiguous() const { return impl_->layout().is_contiguous(); }
  DType dtype() const { return impl_->dtype(); }
  Device device() const { return impl_->device(); }
  void* data() const { return impl_->data(); }
  template <class T> T* data_as() const { return static_cast<T*>(impl_->data()); }
  size_t nbytes() const { return static_cast<size_t>(numel()) * dtype_size(dtype()); }
  StreamHandle stream() const { return Runtime::instance().stream_for(device()); }

  bool requires_grad() const { return impl_->ag().requires_grad; }
  bool is_leaf() const { return !impl_->ag().grad_fn; }
  Tensor grad() const { return impl_->ag().grad ? Tensor(impl_->ag().grad) : Tensor(); }
  const std::shared_ptr<Node>& grad_fn() const { return impl_->ag().grad_fn; }
  Tensor& requires_grad_(bool on);
  void set_grad(const Tensor& g);
  void zero_grad();  // drops the gradient
  void backward(bool retain_graph = false) const;
  void bump_version() const { impl_->buffer()->bump_version(); }
  uint64_t version() const { return impl_->buffer()->version(); }
  bool same_buffer(const Tensor& o) const { return impl_->buffer() == o.impl_->buffer(); }
  // A graph-free alias of the same storage.
  Tensor detach() const;

 private:
  std::shared_ptr<TensorImpl> impl_;
};

// ------------------------------------------------------------------- autograd
struct GraphEdge {
  enum Kind : uint8_t { None, Leaf, Producer, Released };
  Kind kind = None;
  std::shared_ptr<TensorImpl> leaf;  // Leaf
  std::shared_ptr<Node> node;        // Producer
  static GraphEdge capture(const Tensor& t);
};

struct SavedVersion {
  std::shared_ptr<Buffer> buffer;
  uint64_t version;
  const char* role;
};

class Node : public std::enable_shared_from_this<Node> {
 public:
  virtual ~Node() = default;
  virtual const char* name() const = 0;
  // One gradient per input (undefined Tensor = no gradient for that input).
  virtual std::vector<Tensor> backward(const Tensor& grad) = 0;
  // Drops saved tensors once the graph is released.
  virtual void release_saved() {}

  void set_inputs(std::initializer_list<Tensor> inputs);
  void set_inputs(const std::vector<Tensor>& inputs);
  const std::vector<GraphEdge>& edges() const { return edges_; }
  void watch_version(const Tensor& t, const char* role);
  void validate_saved_versions() const;
  bool released() const { return released_; }
  void mark_released();
  // Destination offers, set by the engine around one backward() call: grad_out[i], when defined,
  // is storage with the shape, dtype and device of input i's gradient (a leaf's preassigned
  // gradient slot whose only consumer is this node).  A formula that can write its result there
  // directly does so and returns that tensor for input i; the engine then skips its copy.
  // Formulas that ignore the offer stay correct.
  std::vector<Tensor> grad_out;
  Tensor grad_destination(size_t input) const { return input < grad_out.size() ? grad_out[input] : Tensor(); }
  // Addend offers, also set around one backward() call: grad_addend[i], when defined, is the sum
  // of the gradients that input i's producer has received so far from other consumers.  A
  // formula that can add it while it writes its own result (one pass instead of a separate
  // addition) returns result + addend for input i and calls take_addend(i); the engine then
  // replaces the producer's running sum instead of adding to it.  Ignoring the offer is correct.
  std::vector<Tensor> grad_addend;
  std::vector<char> addend_taken;
  Tensor offered_addend(size_t input) const { return input < grad_addend.size() ? grad_addend[input] : Tensor(); }
  void take_addend(size_t input) { if (input < addend_taken.size()) addend_taken[input] = 1; }
  // Output metadata recorded at attach time, used to validate incoming gradients.
  Shape out_shape;
  DType out_dtype = DType::F32;
  Device out_device;
  // Finalizers registered on the node's output tensor.
  std::vector<std::pair<uint64_t, std::function<void()>>> finalizers;

 private:
  std::vector<GraphEdge> edges_;
  std::vector<SavedVersion> saved_;
  bool released_ = false;
};

bool grad_enabled();
void set_grad_enabled(bool on);
struct NoGradGuard {
  bool prev;
  NoGradGuard() : prev(grad_enabled()) { set_grad_enabled(false); }
  ~NoGradGuard() { set_grad_enabled(prev); }
};

// True when a result computed from these inputs must be attached to the graph.
bool needs_graph(std::initializer_list<Tensor> inputs);
// Marks `out` as produced by `node` (seals edges, records output metadata).
void attach(Tensor& out, std::shared_ptr<Node> node);

struct AutogradEngine {
  static void backward(const Tensor& root, bool retain_graph);
};

}  // namespace ob

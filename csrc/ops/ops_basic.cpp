// Semantic operators, part 1: helpers, arithmetic, unary, shape, cast/to, reductions.
// Formula nodes live next to the operator that attaches them.
//
// Parity (reference project paths): src/ops/{binary,unary,shape,reduce,cast,scalar,fill,
// index,slice,tensor_access}_ops.cpp and include/orthon/autograd/*_node.h.
#include <cmath>
#include <cstring>

#include "ob/kernels.h"
#include "ob/ops.h"

namespace ob {
namespace ops {

void run_kernel(OperatorId op, Device dev, DType dtype, OpCall& call, uint8_t layout) {
  default_dispatcher().run(DispatchRequest{op, dev, dtype, layout}, call);
}

void check_same_device(const Tensor& a, const Tensor& b, const char* op) {
  if (a.device() != b.device())
    throw std::invalid_argument(std::string(op) + ": tensors must be on the same device (got " + a.device().str() +
                                " and " + b.device().str() + ")");
}

void check_same_dtype(const Tensor& a, const Tensor& b, const char* op) {
  if (a.dtype() != b.dtype())
    throw std::invalid_argument(std::string(op) + ": dtype mismatch (" + dtype_name(a.dtype()) + " vs " +
                                dtype_name(b.dtype()) + ")");
}

static uint8_t joint_layout(std::initializer_list<const Tensor*> ts) {
  bool strided = false;
  for (const Tensor* t : ts) {
    if (!t->defined()) continue;
    if (t->numel() == 0) return kEmpty;
    if (!t->is_contiguous()) strided = true;
  }
  return strided ? kStrided : kContiguous;
}

// ------------------------------------------------------------------ raw helpers
void fill_raw(Tensor& t, double value) {
  if (t.numel() == 0) return;
  OpCall c;
  c.in[0] = t;
  c.f[0] = value;
  run_kernel(OperatorId::Fill, t.device(), t.dtype(), c, layout_of(t));
}

static void strided_copy(Tensor& dst, const Tensor& src) {
  if (dst.numel() == 0) return;
  OpCall c;
  c.in[0] = src;
  c.out[0] = dst;
  run_kernel(OperatorId::Contiguous, dst.device(), dst.dtype(), c, joint_layout({&src, &dst}));
}

Tensor clone(const Tensor& t) {
  Tensor out = Tensor::empty(t.shape(), t.dtype(), t.device());
  strided_copy(out, t);
  return out;
}

void copy_(Tensor& dst, const Tensor& src) {
  if (dst.shape() != src.shape()) throw std::invalid_argument("copy_: shape mismatch");
  check_same_dtype(dst, src, "copy_");
  if (dst.device() != src.device()) {
    Tensor moved = to(src, dst.device());
    strided_copy(dst, moved);
  } else {
    strided_copy(dst, src);
  }
  dst.bump_version();
}

void copy_range(Tensor& dst, int64_t dst_off, const Tensor& src, int64_t src_off, int64_t n) {
  check_same_dtype(dst, src, "copy_range");
  check_same_device(dst, src, "copy_range");
  if (!dst.is_contiguous() || !src.is_contiguous()) throw std::invalid_argument("copy_range: tensors must be contiguous");
  if (n < 0 || dst_off < 0 || src_off < 0 || dst_off + n > dst.numel() || src_off + n > src.numel())
    throw std::out_of_range("copy_range: range out of bounds");
  OpCall c;
  c.in[0] = dst;
  c.in[1] = src;
  c.i[0] = dst_off;
  c.i[1] = src_off;
  c.i[2] = n;
  if (n > 0) run_kernel(OperatorId::CopyRange, dst.device(), dst.dtype(), c);
  dst.bump_version();
}

double read_scalar(const Tensor& t, int64_t flat) {
  if (flat < 0 || flat >= t.numel()) throw std::out_of_range("index out of range");
  // Row-major logical index -> element offset.
  int64_t off = 0, rem = flat;
  for (int d = t.ndim() - 1; d >= 0; --d) {
    off += (rem % t.shape()[d]) * t.strides()[d];
    rem /= t.shape()[d];
  }
  Layout one({1}, {1}, t.offset() + off);
  Tensor v = Tensor::view_of(t, one);
  Tensor host = v.device().is_cuda() ? to(v, Device()) : v;
  return load_as_double(host.data(), host.dtype());
}

void write_scalar(Tensor& t, int64_t flat, double value) {
  if (flat < 0 || flat >= t.numel()) throw std::out_of_range("index out of range");
  int64_t off = 0, rem = flat;
  for (int d = t.ndim() - 1; d >= 0; --d) {
    off += (rem % t.shape()[d]) * t.strides()[d];
    rem /= t.shape()[d];
  }
  Layout one({1}, {1}, t.offset() + off);
  Tensor v = Tensor::view_of(t, one);
  fill_raw(v, value);
  t.bump_version();
}

Tensor zeros_like(const Tensor& t) { return Tensor::zeros(t.shape(), t.dtype(), t.device()); }
Tensor ones_like(const Tensor& t) { return Tensor::full(t.shape(), 1.0, t.dtype(), t.device()); }

// ---------------------------------------------------------------------- binary
namespace {

Tensor binary_raw(OperatorId op, const Tensor& a, const Tensor& b, const char* name) {
  check_same_device(a, b, name);
  check_same_dtype(a, b, name);
  default_dispatcher().check_dtype(op, a.device(), a.dtype());
  Tensor out = Tensor::empty(broadcast_shapes(a.shape(), b.shape()), a.dtype(), a.device());
  if (out.numel() == 0) return out;
  OpCall c;
  c.in[0] = a;
  c.in[1] = b;
  c.out[0] = out;
  run_kernel(op, a.device(), a.dtype(), c, joint_layout({&a, &b}));
  return out;
}

struct AddNode : Node {
  Shape sa, sb;
  const char* name() const override { return "AddNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {unbroadcast(g, sa), unbroadcast(g, sb)}; }
};

struct MulNode : Node {
  Tensor a, b;
  const char* name() const override { return "MulNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    return {unbroadcast(mul(g, b), a.shape()), unbroadcast(mul(g, a), b.shape())};
  }
  void release_saved() override { a = Tensor(); b = Tensor(); }
};

struct ScalarNode : Node {
  double scale = 1.0;
  bool is_mul = false;
  const char* name() const override { return is_mul ? "ScalarMulNode" : "ScalarAddNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {is_mul ? mul_scalar(g, scale) : g}; }
};

}  // namespace

Tensor unbroadcast(const Tensor& g, const Shape& target) {
  if (g.shape() == target) return g;
  const int gd = g.ndim(), td = static_cast<int>(target.size());
  if (td > gd) throw std::invalid_argument("unbroadcast: target rank exceeds gradient rank");
  Shape padded(gd, 1);
  for (int i = 0; i < td; ++i) padded[gd - td + i] = target[i];
  for (int i = 0; i < gd; ++i)
    if (padded[i] != g.shape()[i] && padded[i] != 1)
      throw std::invalid_argument("unbroadcast: gradient shape is not a broadcast of the target");
  Tensor gc = contiguous(g);
  Tensor out = Tensor::empty(target, g.dtype(), g.device());
  if (out.numel() == 0) return out;
  OpCall c;
  c.in[0] = gc;
  c.out[0] = out;
  c.list = padded;
  run_kernel(OperatorId::Unbroadcast, g.device(), g.dtype(), c);
  return out;
}

Tensor add(const Tensor& a, const Tensor& b) {
  Tensor out = binary_raw(OperatorId::Add, a, b, "add");
  if (needs_graph({a, b})) {
    auto n = std::make_shared<AddNode>();
    n->sa = a.shape();
    n->sb = b.shape();
    n->set_inputs({a, b});
    attach(out, n);
  }
  return out;
}

Tensor mul(const Tensor& a, const Tensor& b) {
  Tensor out = binary_raw(OperatorId::Mul, a, b, "mul");
  if (needs_graph({a, b})) {
    auto n = std::make_shared<MulNode>();
    n->a = a.detach();
    n->b = b.detach();
    n->watch_version(a, "lhs");
    n->watch_version(b, "rhs");
    n->set_inputs({a, b});
    attach(out, n);
  }
  return out;
}

Tensor sub(const Tensor& a, const Tensor& b) {
  check_same_device(a, b, "sub");
  check_same_dtype(a, b, "sub");
  return add(a, neg(b));
}

Tensor div(const Tensor& a, const Tensor& b) {
  check_same_device(a, b, "div");
  check_same_dtype(a, b, "div");
  return mul(a, reciprocal(b));
}

static Tensor scalar_op(OperatorId op, const Tensor& a, double s, bool is_mul) {
  default_dispatcher().check_dtype(op, a.device(), a.dtype());
  Tensor out = Tensor::empty(a.shape(), a.dtype(), a.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = a;
    c.out[0] = out;
    c.f[0] = s;
    run_kernel(op, a.device(), a.dtype(), c, layout_of(a));
  }
  if (needs_graph({a})) {
    auto n = std::make_shared<ScalarNode>();
    n->scale = s;
    n->is_mul = is_mul;
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor add_scalar(const Tensor& a, double s) { return scalar_op(OperatorId::AddScalar, a, s, false); }
Tensor mul_scalar(const Tensor& a, double s) { return scalar_op(OperatorId::MulScalar, a, s, true); }

// In-place writes are value updates: they bump the buffer version and record no history
// (reference project: src/ops/binary_ops.cpp:128-151, src/ops/fill_ops.cpp:51-61).  A leaf may be
// written at any time (initialisation, optimizers).  A tensor that carries history may not be
// written while gradients are recorded: the write would be invisible to its backward formula.
static void check_inplace_allowed(const Tensor& a, const char* op) {
  if (grad_enabled() && a.requires_grad() && !a.is_leaf())
    throw std::runtime_error(std::string(op) +
                             ": in-place modification of a tensor with autograd history is only allowed under no_grad()");
}

Tensor& add_(Tensor& a, const Tensor& b, double alpha) {
  check_inplace_allowed(a, "add_");
  check_same_device(a, b, "add_");
  check_same_dtype(a, b, "add_");
  if (broadcast_shapes(a.shape(), b.shape()) != a.shape())
    throw std::invalid_argument("add_: source is not broadcastable to the destination shape");
  if (a.same_buffer(b)) {
    const bool identical = a.offset() == b.offset() && a.shape() == b.shape() && a.strides() == b.strides();
    if (!identical) {
      const int64_t a0 = a.offset(), a1 = a.impl()->layout().span_end();
      const int64_t b0 = b.offset(), b1 = b.impl()->layout().span_end();
      if (a0 < b1 && b0 < a1) throw std::invalid_argument("add_: source and destination partially overlap");
    }
  }
  if (a.numel()) {
    OpCall c;
    c.in[0] = a;
    c.in[1] = b;
    c.f[0] = alpha;
    run_kernel(OperatorId::AddInplace, a.device(), a.dtype(), c, joint_layout({&a, &b}));
  }
  a.bump_version();
  return a;
}

Tensor& mul_(Tensor& a, double alpha) {
  check_inplace_allowed(a, "mul_");
  if (a.numel()) {
    OpCall c;
    c.in[0] = a;
    c.f[0] = alpha;
    run_kernel(OperatorId::MulInplace, a.device(), a.dtype(), c, layout_of(a));
  }
  a.bump_version();
  return a;
}

Tensor& fill_(Tensor& a, double v) {
  check_inplace_allowed(a, "fill_");
  fill_raw(a, v);
  a.bump_version();
  return a;
}

// ----------------------------------------------------------------------- unary
namespace {
struct UnaryInfo { OperatorId fwd, bwd; const char* node; };
UnaryInfo unary_info(Unary k) {
  switch (k) {
    case Unary::Neg: return {OperatorId::Neg, OperatorId::Neg, "NegNode"};
    case Unary::Relu: return {OperatorId::Relu, OperatorId::ReluBackward, "ReluNode"};
    case Unary::Sigmoid: return {OperatorId::Sigmoid, OperatorId::SigmoidBackward, "SigmoidNode"};
    case Unary::Tanh: return {OperatorId::Tanh, OperatorId::TanhBackward, "TanhNode"};
    case Unary::LeakyRelu: return {OperatorId::LeakyRelu, OperatorId::LeakyReluBackward, "LeakyReluNode"};
    case Unary::Gelu: return {OperatorId::Gelu, OperatorId::GeluBackward, "GeluNode"};
    case Unary::Exp: return {OperatorId::Exp, OperatorId::ExpBackward, "ExpNode"};
    case Unary::Sqrt: return {OperatorId::Sqrt, OperatorId::SqrtBackward, "SqrtNode"};
    case Unary::Reciprocal: return {OperatorId::Reciprocal, OperatorId::ReciprocalBackward, "ReciprocalNode"};
    case Unary::Log: return {OperatorId::Log, OperatorId::ReciprocalBackward, "LogNode"};
  }
  throw std::logic_error("unknown unary kind");
}

struct UnaryNode : Node {
  Unary kind;
  double param = 0.0;
  Tensor x;
  const char* name() const override { return unary_info(kind).node; }
  std::vector<Tensor> backward(const Tensor& g) override {
    if (kind == Unary::Neg) return {neg(g)};
    if (kind == Unary::Log) return {mul(g, reciprocal(x))};
    return {unary_backward(kind, x, g, param)};
  }
  void release_saved() override { x = Tensor(); }
};
}  // namespace

Tensor unary(Unary kind, const Tensor& a, double param) {
  const UnaryInfo info = unary_info(kind);
  default_dispatcher().check_dtype(info.fwd, a.device(), a.dtype());
  Tensor out = Tensor::empty(a.shape(), a.dtype(), a.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = a;
    c.out[0] = out;
    c.f[0] = param;
    run_kernel(info.fwd, a.device(), a.dtype(), c, layout_of(a));
  }
  if (needs_graph({a})) {
    auto n = std::make_shared<UnaryNode>();
    n->kind = kind;
    n->param = param;
    if (kind != Unary::Neg) {
      n->x = a.detach();
      n->watch_version(a, "input");
    }
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor unary_backward(Unary kind, const Tensor& x, const Tensor& grad, double param) {
  const UnaryInfo info = unary_info(kind);
  check_same_device(x, grad, "unary_backward");
  check_same_dtype(x, grad, "unary_backward");
  if (x.shape() != grad.shape()) throw std::invalid_argument("unary backward: shape mismatch");
  Tensor out = Tensor::empty(x.shape(), x.dtype(), x.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = x;
    c.in[1] = grad;
    c.out[0] = out;
    c.f[0] = param;
    run_kernel(info.bwd, x.device(), x.dtype(), c, joint_layout({&x, &grad}));
  }
  return out;
}

Tensor dropout_mask(const Shape& shape, double p, uint64_t seed, DType dtype, Device dev) {
  if (!(p >= 0.0 && p < 1.0)) throw std::invalid_argument("dropout: p must be in [0, 1)");
  Tensor mask = Tensor::empty(shape, dtype, dev);
  if (mask.numel()) {
    OpCall c;
    c.out[0] = mask;
    c.f[0] = p;
    c.i[0] = static_cast<int64_t>(seed);
    run_kernel(OperatorId::DropoutMask, dev, dtype, c);
  }
  return mask;
}

namespace {
Tensor dropout_apply_cuda(const Tensor& x, double p, uint64_t seed) {
  Tensor out = Tensor::empty(x.shape(), x.dtype(), x.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = x;
    c.out[0] = out;
    c.f[0] = p;
    c.i[0] = static_cast<int64_t>(seed);
    run_kernel(OperatorId::DropoutMask, x.device(), x.dtype(), c);
  }
  return out;
}
// Backward of the fused CUDA dropout: the same mask, recomputed from (p, seed), applied to the gradient.
struct DropoutNode : Node {
  double p = 0.0;
  uint64_t seed = 0;
  const char* name() const override { return "DropoutNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {dropout_apply_cuda(contiguous(g), p, seed)}; }
};
}  // namespace

// CPU: mask tensor times input (reference project: src/ops/unary_ops.cpp:150-166).  CUDA: one
// fused pass over a packed input, same random stream, no mask tensor kept for backward.
Tensor dropout(const Tensor& a, double p, uint64_t seed) {
  if (!a.device().is_cuda()) {
    Tensor mask = dropout_mask(a.shape(), p, seed, a.dtype(), a.device());
    return mul(a, mask);
  }
  if (!(p >= 0.0 && p < 1.0)) throw std::invalid_argument("dropout: p must be in [0, 1)");
  default_dispatcher().check_dtype(OperatorId::DropoutMask, a.device(), a.dtype());
  Tensor x = a;
  if (!a.is_contiguous()) {
    NoGradGuard guard;
    x = contiguous(a);
  }
  Tensor out = dropout_apply_cuda(x, p, seed);
  if (needs_graph({a})) {
    auto n = std::make_shared<DropoutNode>();
    n->p = p;
    n->seed = seed;
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

// ----------------------------------------------------------------------- shape
namespace {
struct ReshapeNode : Node {
  Shape in_shape;
  const char* name() const override { return "ReshapeNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {reshape(contiguous(g), in_shape)}; }
};
struct TransposeNode : Node {
  int d0, d1;
  const char* name() const override { return "TransposeNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {transpose(g, d0, d1)}; }
};
struct ContiguousNode : Node {
  const char* name() const override { return "ContiguousNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {g}; }
};
struct SliceNode : Node {
  Shape in_shape;
  int dim;
  int64_t start, end;
  const char* name() const override { return "SliceNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor z = Tensor::zeros(in_shape, g.dtype(), g.device());
    Tensor view = slice(z, dim, start, end);
    copy_(view, g);
    return {z};
  }
};
struct IndexNode : Node {
  Shape in_shape;
  int64_t i;
  const char* name() const override { return "IndexNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor z = Tensor::zeros(in_shape, g.dtype(), g.device());
    Tensor view = index(z, i);
    copy_(view, g);
    return {z};
  }
};
struct CastNode : Node {
  DType src;
  const char* name() const override { return "CastNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {cast(g, src)}; }
};
struct ToNode : Node {
  Device src;
  const char* name() const override { return "ToNode"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {to(g, src)}; }
};
}  // namespace

Tensor reshape(const Tensor& a, const Shape& shape_in) {
  Shape shape = shape_in;
  int infer = -1;
  int64_t known = 1;
  for (size_t i = 0; i < shape.size(); ++i) {
    if (shape[i] == -1) {
      if (infer >= 0) throw std::invalid_argument("reshape: only one dimension can be inferred");
      infer = static_cast<int>(i);
    } else if (shape[i] < 0) {
      throw std::invalid_argument("reshape: negative extent");
    } else {
      known *= shape[i];
    }
  }
  if (infer >= 0) {
    if (known == 0 || a.numel() % known != 0) throw std::invalid_argument("reshape: cannot infer the missing extent");
    shape[infer] = a.numel() / known;
  }
  if (Layout::checked_numel(shape) != a.numel())
    throw std::invalid_argument("reshape: cannot reshape " + shape_str(a.shape()) + " to " + shape_str(shape));
  if (!a.is_contiguous()) throw std::invalid_argument("reshape: tensor must be contiguous; call contiguous() first");
  Tensor out = Tensor::view_of(a, Layout(shape, Layout::contiguous_strides(shape), a.offset()));
  if (needs_graph({a})) {
    auto n = std::make_shared<ReshapeNode>();
    n->in_shape = a.shape();
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor flatten(const Tensor& a, int start, int end) {
  const int nd = a.ndim();
  if (nd == 0) return reshape(a, {1});
  if (start < 0) start += nd;
  if (end < 0) end += nd;
  if (start < 0 || end >= nd || start > end) throw std::invalid_argument("flatten: invalid dimension range");
  Shape s;
  for (int i = 0; i < start; ++i) s.push_back(a.shape()[i]);
  int64_t m = 1;
  for (int i = start; i <= end; ++i) m *= a.shape()[i];
  s.push_back(m);
  for (int i = end + 1; i < nd; ++i) s.push_back(a.shape()[i]);
  return reshape(contiguous(a), s);
}

Tensor transpose(const Tensor& a, int d0, int d1) {
  const int nd = a.ndim();
  if (d0 < 0) d0 += nd;
  if (d1 < 0) d1 += nd;
  if (d0 < 0 || d0 >= nd || d1 < 0 || d1 >= nd) throw std::invalid_argument("transpose: dimension out of range");
  Shape s = a.shape(), st = a.strides();
  std::swap(s[d0], s[d1]);
  std::swap(st[d0], st[d1]);
  Tensor out = Tensor::view_of(a, Layout(s, st, a.offset()));
  if (needs_graph({a})) {
    auto n = std::make_shared<TransposeNode>();
    n->d0 = d0;
    n->d1 = d1;
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor contiguous(const Tensor& a) {
  if (a.is_contiguous()) return a;
  Tensor out = clone(a);
  if (needs_graph({a})) {
    auto n = std::make_shared<ContiguousNode>();
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor slice(const Tensor& a, int dim, int64_t start, int64_t end) {
  const int nd = a.ndim();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) throw std::invalid_argument("slice: dimension out of range");
  const int64_t n = a.shape()[dim];
  if (start < 0) start += n;
  if (end < 0) end += n;
  if (start < 0 || end > n || start > end) throw std::out_of_range("slice: range out of bounds");
  Shape s = a.shape();
  s[dim] = end - start;
  Tensor out = Tensor::view_of(a, Layout(s, a.strides(), a.offset() + start * a.strides()[dim]));
  if (needs_graph({a})) {
    auto node = std::make_shared<SliceNode>();
    node->in_shape = a.shape();
    node->dim = dim;
    node->start = start;
    node->end = end;
    node->set_inputs({a});
    attach(out, node);
  }
  return out;
}

Tensor index(const Tensor& a, int64_t i) {
  if (a.ndim() == 0) throw std::invalid_argument("index: cannot index a rank-0 tensor");
  const int64_t n = a.shape()[0];
  if (i < 0) i += n;
  if (i < 0 || i >= n) throw std::out_of_range("index out of range");
  Shape s(a.shape().begin() + 1, a.shape().end()), st(a.strides().begin() + 1, a.strides().end());
  if (s.empty()) { s = {1}; st = {1}; }
  Tensor out = Tensor::view_of(a, Layout(s, st, a.offset() + i * a.strides()[0]));
  if (needs_graph({a})) {
    auto node = std::make_shared<IndexNode>();
    node->in_shape = a.shape();
    node->i = i;
    node->set_inputs({a});
    attach(out, node);
  }
  return out;
}

Tensor cast(const Tensor& a, DType dtype) {
  if (a.dtype() == dtype) return contiguous(a);
  default_dispatcher().check_dtype(OperatorId::Cast, a.device(), a.dtype());
  Tensor out = Tensor::empty(a.shape(), dtype, a.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = a;
    c.out[0] = out;
    run_kernel(OperatorId::Cast, a.device(), a.dtype(), c, layout_of(a));
  }
  if (needs_graph({a}) && dtype_is_floating(dtype) && dtype_is_floating(a.dtype())) {
    auto n = std::make_shared<CastNode>();
    n->src = a.dtype();
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

Tensor to(const Tensor& a, Device dev) {
  if (dev.is_cuda()) Runtime::instance().cuda(dev.index);  // validates the ordinal
  Tensor out = Tensor::empty(a.shape(), a.dtype(), dev);
  if (out.numel()) {
    OpCall c;
    c.in[0] = a;
    c.out[0] = out;
    // Transfers are owned by the backend of whichever side is a device.
    const Device owner = a.device().is_cuda() ? a.device() : dev;
    run_kernel(OperatorId::To, owner, a.dtype(), c, layout_of(a));
  }
  if (needs_graph({a}) && dtype_is_floating(a.dtype())) {
    auto n = std::make_shared<ToNode>();
    n->src = a.device();
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

// ------------------------------------------------------------------ reductions
namespace {

struct ReductionPlan {
  int64_t outer = 1, reduce = 1, inner = 1;
  Shape out_shape, keep_shape;
};

// Normalizes an optional dim (negatives allowed) into outer/reduce/inner extents.
// (reference project: src/reduction/reduction.cpp:45-105)
ReductionPlan plan_reduction(const Tensor& a, std::optional<int> dim, bool keepdim, const char* op) {
  if (a.numel() == 0) throw std::invalid_argument(std::string(op) + ": cannot reduce an empty tensor");
  ReductionPlan p;
  const int nd = a.ndim();
  if (!dim.has_value()) {
    p.reduce = a.numel();
    p.keep_shape = Shape(nd == 0 ? 1 : nd, 1);
    p.out_shape = keepdim ? p.keep_shape : Shape{1};
    return p;
  }
  int d = *dim;
  if (d < 0) d += nd;
  if (d < 0 || d >= nd) throw std::invalid_argument(std::string(op) + ": dimension out of range");
  for (int i = 0; i < d; ++i) p.outer *= a.shape()[i];
  p.reduce = a.shape()[d];
  for (int i = d + 1; i < nd; ++i) p.inner *= a.shape()[i];
  p.keep_shape = a.shape();
  p.keep_shape[d] = 1;
  if (keepdim) {
    p.out_shape = p.keep_shape;
  } else {
    for (int i = 0; i < nd; ++i)
      if (i != d) p.out_shape.push_back(a.shape()[i]);
    if (p.out_shape.empty()) p.out_shape = {1};
  }
  return p;
}

struct ReduceNode : Node {
  Shape in_shape, keep_shape;
  double scale = 1.0;
  bool is_mean = false;
  const char* name() const override { return is_mean ? "MeanNode" : "SumNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gk = reshape(contiguous(g), keep_shape);
    Tensor grad = add(Tensor::zeros(in_shape, g.dtype(), g.device()), gk);
    if (scale != 1.0) grad = mul_scalar(grad, scale);
    return {grad};
  }
};

struct MaxNode : Node {
  Shape in_shape;
  Tensor indices;
  int64_t outer, reduce, inner;
  const char* name() const override { return "MaxNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor out = Tensor::empty(in_shape, g.dtype(), g.device());
    OpCall c;
    c.in[0] = contiguous(g);
    c.in[1] = indices;
    c.out[0] = out;
    c.i[0] = outer;
    c.i[1] = reduce;
    c.i[2] = inner;
    run_kernel(OperatorId::MaxBackward, g.device(), g.dtype(), c);
    return {out};
  }
  void release_saved() override { indices = Tensor(); }
};

Tensor reduce_impl(const Tensor& a, std::optional<int> dim, bool keepdim, bool is_mean) {
  const OperatorId op = is_mean ? OperatorId::Mean : OperatorId::Sum;
  default_dispatcher().check_dtype(op, a.device(), a.dtype());
  const ReductionPlan p = plan_reduction(a, dim, keepdim, is_mean ? "mean" : "sum");
  Tensor ac = contiguous(a.detach());
  Tensor out = Tensor::empty(p.out_shape, a.dtype(), a.device());
  OpCall c;
  c.in[0] = ac;
  c.out[0] = out;
  c.i[0] = p.outer;
  c.i[1] = p.reduce;
  c.i[2] = p.inner;
  run_kernel(op, a.device(), a.dtype(), c);
  if (needs_graph({a})) {
    auto n = std::make_shared<ReduceNode>();
    n->in_shape = a.shape();
    n->keep_shape = p.keep_shape;
    n->is_mean = is_mean;
    n->scale = is_mean ? 1.0 / static_cast<double>(p.reduce) : 1.0;
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

}  // namespace

Tensor sum(const Tensor& a, std::optional<int> dim, bool keepdim) { return reduce_impl(a, dim, keepdim, false); }
Tensor mean(const Tensor& a, std::optional<int> dim, bool keepdim) { return reduce_impl(a, dim, keepdim, true); }

std::pair<Tensor, Tensor> max(const Tensor& a, std::optional<int> dim, bool keepdim) {
  default_dispatcher().check_dtype(OperatorId::Max, a.device(), a.dtype());
  const ReductionPlan p = plan_reduction(a, dim, keepdim, "max");
  Tensor ac = contiguous(a.detach());
  Tensor values = Tensor::empty(p.out_shape, a.dtype(), a.device());
  Tensor indices = Tensor::empty(p.out_shape, DType::I64, a.device());
  OpCall c;
  c.in[0] = ac;
  c.out[0] = values;
  c.out[1] = indices;
  c.i[0] = p.outer;
  c.i[1] = p.reduce;
  c.i[2] = p.inner;
  run_kernel(OperatorId::Max, a.device(), a.dtype(), c);
  if (needs_graph({a})) {
    auto n = std::make_shared<MaxNode>();
    n->in_shape = a.shape();
    n->indices = indices;
    n->outer = p.outer;
    n->reduce = p.reduce;
    n->inner = p.inner;
    n->set_inputs({a});
    attach(values, n);
  }
  return {values, indices};
}

Tensor argmax(const Tensor& a, std::optional<int> dim, bool keepdim) {
  NoGradGuard g;
  return max(a, dim, keepdim).second;
}

void isfinite_into(const Tensor& a, Tensor& flag) {
  if (flag.dtype() != DType::I32 || flag.numel() != 1 || flag.device() != a.device())
    throw std::invalid_argument("isfinite_into: flag must be a one-element int32 tensor on the same device");
  if (a.numel() == 0) return;
  OpCall c;
  c.in[0] = a;
  c.in[1] = flag;
  run_kernel(OperatorId::IsFiniteAll, a.device(), a.dtype(), c, layout_of(a));
}

bool isfinite_all(const Tensor& a) {
  if (a.numel() == 0) return true;
  OpCall c;
  c.in[0] = a;
  run_kernel(OperatorId::IsFiniteAll, a.device(), a.dtype(), c, layout_of(a));
  return c.i[0] != 0;
}

}  // namespace ops
}  // namespace ob

// Semantic operators, part 2: GEMM family, softmax/losses, embedding, conv/pool,
// LayerNorm, attention, AMP helpers and fused optimizer updates.
//
// Parity (reference project paths): src/ops/{matmul,fusion,softmax,cross_entropy,
// nll_loss,embedding,conv2d,maxpool2d,tensor_access}_ops.cpp,
// include/orthon/planning/{conv2d,maxpool2d,index}_validation.h,
// python/orthon/functional/math.py:39-72 (attention), python/orthon/nn/layernorm.py:34-61.
#include <cmath>

#include "ob/kernels.h"
#include "ob/ops.h"

namespace ob {
namespace ops {

// ------------------------------------------------------------------------ GEMM
namespace {

Tensor gemm_raw(const Tensor& a, bool ta, const Tensor& b, bool tb, const Tensor& destination = Tensor()) {
  check_same_device(a, b, "matmul");
  check_same_dtype(a, b, "matmul");
  default_dispatcher().check_dtype(OperatorId::Matmul, a.device(), a.dtype());
  const int nd = a.ndim();
  if (nd != b.ndim() || nd < 2 || nd > 4)
    throw std::invalid_argument("matmul: operands must both be 2-D, 3-D or 4-D (got " + shape_str(a.shape()) +
                                " and " + shape_str(b.shape()) + ")");
  for (int i = 0; i < nd - 2; ++i)
    if (a.shape()[i] != b.shape()[i])
      throw std::invalid_argument("matmul: batch dimensions must match (got " + shape_str(a.shape()) + " and " +
                                  shape_str(b.shape()) + ")");
  const int64_t M = ta ? a.shape()[nd - 1] : a.shape()[nd - 2];
  const int64_t K = ta ? a.shape()[nd - 2] : a.shape()[nd - 1];
  const int64_t Kb = tb ? b.shape()[nd - 1] : b.shape()[nd - 2];
  const int64_t N = tb ? b.shape()[nd - 2] : b.shape()[nd - 1];
  if (K != Kb)
    throw std::invalid_argument("matmul: inner dimensions do not match (" + shape_str(a.shape()) + " @ " +
                                shape_str(b.shape()) + ")");
  Shape os(a.shape().begin(), a.shape().end() - 2);
  os.push_back(M);
  os.push_back(N);
  // A caller-provided destination (a contiguous tensor of the result's shape, dtype and device:
  // a leaf's gradient slot offered by the engine) takes the product directly.
  const bool direct = destination.defined() && destination.shape() == os && destination.dtype() == a.dtype() &&
                      destination.device() == a.device() && destination.is_contiguous();
  Tensor out = direct ? destination : Tensor::empty(os, a.dtype(), a.device());
  if (out.numel() == 0) return out;
  if (K == 0) {
    fill_raw(out, 0.0);
    return out;
  }
  OpCall c;
  c.in[0] = a;
  c.in[1] = b;
  c.out[0] = out;
  c.i[0] = ta;
  c.i[1] = tb;
  const bool strided = !a.is_contiguous() || !b.is_contiguous();
  run_kernel(OperatorId::Matmul, a.device(), a.dtype(), c, strided ? kStrided : kContiguous);
  return out;
}

struct MatMulNode : Node {
  Tensor a, b;
  bool ta, tb;
  const char* name() const override { return "MatMulNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor da = ta ? gemm_raw(b, tb, g, true, grad_destination(0)) : gemm_raw(g, false, b, !tb, grad_destination(0));
    Tensor db = tb ? gemm_raw(g, true, a, ta, grad_destination(1)) : gemm_raw(a, !ta, g, false, grad_destination(1));
    return {da, db};
  }
  void release_saved() override { a = Tensor(); b = Tensor(); }
};

}  // namespace

Tensor gemm(const Tensor& a, bool ta, const Tensor& b, bool tb) {
  Tensor out = gemm_raw(a, ta, b, tb);
  if (needs_graph({a, b})) {
    auto n = std::make_shared<MatMulNode>();
    n->a = a.detach();
    n->b = b.detach();
    n->ta = ta;
    n->tb = tb;
    n->watch_version(a, "lhs");
    n->watch_version(b, "rhs");
    n->set_inputs({a, b});
    attach(out, n);
  }
  return out;
}

Tensor matmul(const Tensor& a, const Tensor& b) {
  if (!(a.ndim() == b.ndim() && (a.ndim() == 2 || a.ndim() == 3)))
    throw std::invalid_argument("matmul: expected 2-D @ 2-D or batched 3-D @ 3-D operands (got " +
                                shape_str(a.shape()) + " and " + shape_str(b.shape()) + ")");
  return gemm(a, false, b, false);
}

namespace {
struct LinearNode : Node {
  Tensor x2, w, saved_act;  // saved_act: pre-activation (GELU) or output (ReLU)
  Act act;
  bool has_bias, has_res;
  Shape x_shape;
  const char* name() const override { return "LinearNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const int64_t N = w.shape()[1];
    Tensor g2 = reshape(contiguous(g), {-1, N});
    Tensor gz = g2;
    if (act == Act::Relu) gz = unary_backward(Unary::Relu, saved_act, g2);
    else if (act == Act::Gelu) gz = unary_backward(Unary::Gelu, saved_act, g2);
    Tensor dx = reshape(gemm_raw(gz, false, w, true), x_shape);
    Tensor dw = gemm_raw(x2, true, gz, false, grad_destination(1));
    std::vector<Tensor> out{dx, dw};
    out.push_back(has_bias ? sum(gz, 0, false) : Tensor());
    out.push_back(has_res ? g : Tensor());
    return out;
  }
  void release_saved() override { x2 = Tensor(); w = Tensor(); saved_act = Tensor(); }
};
}  // namespace

Tensor linear(const Tensor& x, const Tensor& w, const Tensor& b, Act act, const Tensor& residual) {
  check_same_device(x, w, "linear");
  check_same_dtype(x, w, "linear");
  if (w.ndim() != 2) throw std::invalid_argument("linear: weight must be 2-D [in, out]");
  if (x.ndim() < 1 || x.shape().back() != w.shape()[0])
    throw std::invalid_argument("linear: input features " + shape_str(x.shape()) + " do not match weight " +
                                shape_str(w.shape()));
  const int64_t K = w.shape()[0], N = w.shape()[1];
  if (b.defined()) {
    check_same_device(x, b, "linear");
    check_same_dtype(x, b, "linear");
    if (b.ndim() != 1 || b.shape()[0] != N) throw std::invalid_argument("linear: bias must have shape [out]");
  }
  Shape os(x.shape().begin(), x.shape().end() - 1);
  os.push_back(N);
  if (residual.defined()) {
    check_same_device(x, residual, "linear");
    check_same_dtype(x, residual, "linear");
    if (residual.shape() != os) throw std::invalid_argument("linear: residual shape must match the output");
  }
  default_dispatcher().check_dtype(OperatorId::Linear, x.device(), x.dtype());
  Tensor x2 = reshape(contiguous(x.detach()), {-1, K});
  Tensor wc = w.detach();
  Tensor out = Tensor::empty(os, x.dtype(), x.device());
  const bool graph = needs_graph({x, w, b, residual});
  Tensor preact;
  if (out.numel()) {
    OpCall c;
    c.in[0] = x2;
    c.in[1] = wc;
    if (b.defined()) c.in[2] = b.detach();
    if (residual.defined()) c.in[3] = contiguous(residual.detach());
    c.out[0] = Tensor::view_of(out, Layout(Shape{x2.shape()[0], N}));
    if (graph && act == Act::Gelu) {
      preact = Tensor::empty({x2.shape()[0], N}, x.dtype(), x.device());
      c.out[1] = preact;
    }
    c.i[0] = static_cast<int>(act);
    run_kernel(OperatorId::Linear, x.device(), x.dtype(), c, wc.is_contiguous() ? kContiguous : kStrided);
  }
  if (graph) {
    auto n = std::make_shared<LinearNode>();
    n->x2 = x2;
    n->w = wc;
    n->act = act;
    n->has_bias = b.defined();
    n->has_res = residual.defined();
    n->x_shape = x.shape();
    if (act == Act::Gelu) n->saved_act = preact;
    if (act == Act::Relu) {
      if (residual.defined()) throw std::invalid_argument("linear: ReLU with a residual is not differentiable here");
      n->saved_act = Tensor::view_of(out, Layout(Shape{x2.shape()[0], N}));
    }
    n->watch_version(x, "input");
    n->watch_version(w, "weight");
    n->set_inputs({x, w, b, residual});
    attach(out, n);
  }
  return out;
}

namespace {
// One raw Linear kernel call: y = act(x2 @ w + b) (+ aux), optional pre-activation output.
// act 3 multiplies by aux instead of adding it; act 4 is GELU whose second output is the
// derivative gelu'(pre-activation) instead of the pre-activation.
void linear_raw(const Tensor& x2, const Tensor& w, const Tensor& b, int act, const Tensor& aux, Tensor& y, Tensor* preact) {
  OpCall c;
  c.in[0] = x2;
  c.in[1] = w;
  if (b.defined()) c.in[2] = b;
  if (aux.defined()) c.in[3] = aux;
  c.out[0] = y;
  if (preact) c.out[1] = *preact;
  c.i[0] = act;
  run_kernel(OperatorId::Linear, x2.device(), x2.dtype(), c, w.is_contiguous() ? kContiguous : kStrided);
}

struct MlpNode : Node {
  Tensor x2, w1, w2, z, h;
  bool has_b1, has_b2, has_res;
  Shape x_shape;
  const char* name() const override { return "MlpGeluNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const int64_t E = w2.shape()[1], F = w1.shape()[1];
    Tensor g2 = reshape(contiguous(g), {-1, E});
    // dz = (g @ w2^T) * gelu'(z) in one GEMM (z holds the derivative saved by the forward).
    Tensor dz = Tensor::empty({g2.shape()[0], F}, g2.dtype(), g2.device());
    linear_raw(g2, transpose(w2, 0, 1), Tensor(), 3, z, dz, nullptr);
    Tensor dw2 = gemm_raw(h, true, g2, false, grad_destination(3));
    Tensor dx = reshape(gemm_raw(dz, false, w1, true), x_shape);
    Tensor dw1 = gemm_raw(x2, true, dz, false, grad_destination(1));
    std::vector<Tensor> out{dx, dw1, has_b1 ? sum(dz, 0, false) : Tensor(), dw2, has_b2 ? sum(g2, 0, false) : Tensor(),
                            has_res ? g : Tensor()};
    return out;
  }
  void release_saved() override { x2 = Tensor(); w1 = Tensor(); w2 = Tensor(); z = Tensor(); h = Tensor(); }
};
}  // namespace

Tensor mlp_gelu(const Tensor& x, const Tensor& w1, const Tensor& b1, const Tensor& w2, const Tensor& b2, const Tensor& residual) {
  if (!needs_graph({x, w1, b1, w2, b2, residual}))
    return linear(linear(x, w1, b1, Act::Gelu, Tensor()), w2, b2, Act::None, residual);
  check_same_device(x, w1, "mlp_gelu");
  check_same_device(x, w2, "mlp_gelu");
  check_same_dtype(x, w1, "mlp_gelu");
  check_same_dtype(x, w2, "mlp_gelu");
  if (w1.ndim() != 2 || w2.ndim() != 2 || x.ndim() < 1 || x.shape().back() != w1.shape()[0] || w1.shape()[1] != w2.shape()[0])
    throw std::invalid_argument("mlp_gelu: expected x [..., in], w1 [in, hidden], w2 [hidden, out]");
  const int64_t K = w1.shape()[0], F = w1.shape()[1], E = w2.shape()[1];
  if ((b1.defined() && (b1.ndim() != 1 || b1.shape()[0] != F)) || (b2.defined() && (b2.ndim() != 1 || b2.shape()[0] != E)))
    throw std::invalid_argument("mlp_gelu: bias shapes must be [hidden] and [out]");
  Shape os(x.shape().begin(), x.shape().end() - 1);
  os.push_back(E);
  if (residual.defined() && residual.shape() != os) throw std::invalid_argument("mlp_gelu: residual shape must match the output");
  default_dispatcher().check_dtype(OperatorId::Linear, x.device(), x.dtype());
  Tensor x2 = reshape(contiguous(x.detach()), {-1, K});
  const int64_t M = x2.shape()[0];
  Tensor z = Tensor::empty({M, F}, x.dtype(), x.device()), h = Tensor::empty({M, F}, x.dtype(), x.device());
  Tensor out = Tensor::empty(os, x.dtype(), x.device());
  Tensor w1c = w1.detach(), w2c = w2.detach();
  if (out.numel()) {
    linear_raw(x2, w1c, b1.defined() ? b1.detach() : Tensor(), 4, Tensor(), h, &z);
    Tensor out2 = Tensor::view_of(out, Layout(Shape{M, E}));
    linear_raw(h, w2c, b2.defined() ? b2.detach() : Tensor(), 0,
               residual.defined() ? reshape(contiguous(residual.detach()), {M, E}) : Tensor(), out2, nullptr);
  }
  auto n = std::make_shared<MlpNode>();
  n->x2 = x2; n->w1 = w1c; n->w2 = w2c; n->z = z; n->h = h;
  n->has_b1 = b1.defined(); n->has_b2 = b2.defined(); n->has_res = residual.defined();
  n->x_shape = x.shape();
  n->watch_version(x, "input");
  n->watch_version(w1, "first weight");
  n->watch_version(w2, "second weight");
  n->set_inputs({x, w1, b1, w2, b2, residual});
  attach(out, n);
  return out;
}

Tensor fused_linear_relu(const Tensor& x, const Tensor& w, const Tensor& b) {
  if (x.ndim() != 2) throw std::invalid_argument("fused_linear_relu: input must be 2-D");
  return linear(x, w, b, Act::Relu, Tensor());
}

// ------------------------------------------------------------- softmax family
namespace {
struct Orp { int64_t outer = 1, reduce = 1, inner = 1; };
Orp split_dim(const Tensor& a, int& dim, const char* op) {
  const int nd = a.ndim();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) throw std::invalid_argument(std::string(op) + ": dimension out of range");
  Orp p;
  for (int i = 0; i < dim; ++i) p.outer *= a.shape()[i];
  p.reduce = a.shape()[dim];
  for (int i = dim + 1; i < nd; ++i) p.inner *= a.shape()[i];
  return p;
}

struct SoftmaxNode : Node {
  Tensor y;
  Orp p;
  bool log_form;
  const char* name() const override { return log_form ? "LogSoftmaxNode" : "SoftmaxNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor out = Tensor::empty(y.shape(), y.dtype(), y.device());
    OpCall c;
    c.in[0] = y;
    c.in[1] = contiguous(g);
    c.out[0] = out;
    c.i[0] = p.outer;
    c.i[1] = p.reduce;
    c.i[2] = p.inner;
    run_kernel(log_form ? OperatorId::LogSoftmaxBackward : OperatorId::SoftmaxBackward, y.device(), y.dtype(), c);
    return {out};
  }
  void release_saved() override { y = Tensor(); }
};

Tensor softmax_impl(const Tensor& a, int dim, bool log_form) {
  const OperatorId op = log_form ? OperatorId::LogSoftmax : OperatorId::Softmax;
  default_dispatcher().check_dtype(op, a.device(), a.dtype());
  if (a.numel() == 0) throw std::invalid_argument("softmax: empty tensor");
  const Orp p = split_dim(a, dim, log_form ? "log_softmax" : "softmax");
  Tensor ac = contiguous(a.detach());
  Tensor out = Tensor::empty(a.shape(), a.dtype(), a.device());
  OpCall c;
  c.in[0] = ac;
  c.out[0] = out;
  c.i[0] = p.outer;
  c.i[1] = p.reduce;
  c.i[2] = p.inner;
  run_kernel(op, a.device(), a.dtype(), c);
  if (needs_graph({a})) {
    auto n = std::make_shared<SoftmaxNode>();
    n->y = out.detach();
    n->p = p;
    n->log_form = log_form;
    n->watch_version(out, "output");
    n->set_inputs({a});
    attach(out, n);
  }
  return out;
}

void check_targets_host(const Tensor& targets, int64_t classes, const char* op) {
  // Host tensors are validated eagerly; device targets are range-checked inside the kernels,
  // which clamp and raise the device error flag instead of faulting.
  if (!targets.device().is_cpu()) return;
  const int64_t n = targets.numel();
  for (int64_t i = 0; i < n; ++i) {
    const int64_t t = targets.dtype() == DType::I64 ? targets.data_as<int64_t>()[i]
                                                    : static_cast<int64_t>(targets.data_as<int32_t>()[i]);
    if (t < 0 || t >= classes)
      throw std::out_of_range(std::string(op) + ": target " + std::to_string(t) + " is out of range for " +
                              std::to_string(classes) + " classes");
  }
}

Tensor prepare_targets(const Tensor& targets, const Tensor& like, int64_t rows, const char* op) {
  if (targets.dtype() != DType::I64 && targets.dtype() != DType::I32)
    throw std::invalid_argument(std::string(op) + ": targets must be int32 or int64");
  if (targets.numel() != rows) throw std::invalid_argument(std::string(op) + ": target count must match the batch");
  Tensor t = contiguous(targets);
  if (t.device() != like.device()) t = to(t, like.device());
  return t;
}

struct CrossEntropyNode : Node {
  Tensor logits, targets, lse;
  const char* name() const override { return "CrossEntropyNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor out = Tensor::empty(logits.shape(), logits.dtype(), logits.device());
    OpCall c;
    c.in[0] = logits;
    c.in[1] = targets;
    c.in[2] = contiguous(g);
    c.in[3] = lse;
    c.out[0] = out;
    run_kernel(OperatorId::CrossEntropyBackward, logits.device(), logits.dtype(), c);
    return {out};
  }
  void release_saved() override { logits = Tensor(); targets = Tensor(); lse = Tensor(); }
};

struct NllNode : Node {
  Tensor targets;
  Shape in_shape;
  int reduction;
  const char* name() const override { return "NllLossNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor out = Tensor::empty(in_shape, g.dtype(), g.device());
    OpCall c;
    c.in[0] = contiguous(g);
    c.in[1] = targets;
    c.out[0] = out;
    c.i[0] = reduction;
    run_kernel(OperatorId::NllLossBackward, g.device(), g.dtype(), c);
    return {out};
  }
  void release_saved() override { targets = Tensor(); }
};
}  // namespace

Tensor softmax(const Tensor& a, int dim) { return softmax_impl(a, dim, false); }
Tensor log_softmax(const Tensor& a, int dim) { return softmax_impl(a, dim, true); }

Tensor cross_entropy(const Tensor& logits, const Tensor& targets) {
  if (logits.ndim() != 2) throw std::invalid_argument("cross_entropy: logits must be 2-D [batch, classes]");
  if (logits.numel() == 0) throw std::invalid_argument("cross_entropy: empty logits");
  default_dispatcher().check_dtype(OperatorId::CrossEntropy, logits.device(), logits.dtype());
  check_targets_host(targets, logits.shape()[1], "cross_entropy");
  Tensor t = prepare_targets(targets, logits, logits.shape()[0], "cross_entropy");
  Tensor lc = contiguous(logits.detach());
  // The mean loss is kept in float32 for low-precision logits.
  const DType loss_dtype = dtype_is_low_precision(logits.dtype()) ? DType::F32 : logits.dtype();
  Tensor loss = Tensor::empty({1}, loss_dtype, logits.device());
  Tensor lse = Tensor::empty({logits.shape()[0]}, DType::F32, logits.device());
  OpCall c;
  c.in[0] = lc;
  c.in[1] = t;
  c.out[0] = loss;
  c.out[1] = lse;
  run_kernel(OperatorId::CrossEntropy, logits.device(), logits.dtype(), c);
  if (needs_graph({logits})) {
    auto n = std::make_shared<CrossEntropyNode>();
    n->logits = lc;
    n->targets = t;
    n->lse = lse;
    n->watch_version(logits, "logits");
    n->set_inputs({logits});
    attach(loss, n);
  }
  return loss;
}

Tensor cross_entropy_host(const Tensor& logits, const std::vector<int64_t>& targets) {
  Tensor t = Tensor::empty({static_cast<int64_t>(targets.size())}, DType::I64, Device());
  for (size_t i = 0; i < targets.size(); ++i) t.data_as<int64_t>()[i] = targets[i];
  return cross_entropy(logits, t);
}

Tensor nll_loss(const Tensor& lp, const Tensor& targets, const std::string& reduction) {
  if (lp.ndim() != 2) throw std::invalid_argument("nll_loss: log-probabilities must be 2-D [N, C]");
  if (lp.numel() == 0) throw std::invalid_argument("nll_loss: empty input");
  int red;
  if (reduction == "none") red = 0;
  else if (reduction == "mean") red = 1;
  else if (reduction == "sum") red = 2;
  else throw std::invalid_argument("nll_loss: reduction must be 'none', 'mean' or 'sum'");
  default_dispatcher().check_dtype(OperatorId::NllLoss, lp.device(), lp.dtype());
  check_targets_host(targets, lp.shape()[1], "nll_loss");
  Tensor t = prepare_targets(targets, lp, lp.shape()[0], "nll_loss");
  Tensor lc = contiguous(lp.detach());
  Tensor out = Tensor::empty(red == 0 ? Shape{lp.shape()[0]} : Shape{1}, lp.dtype(), lp.device());
  OpCall c;
  c.in[0] = lc;
  c.in[1] = t;
  c.out[0] = out;
  c.i[0] = red;
  run_kernel(OperatorId::NllLoss, lp.device(), lp.dtype(), c);
  if (needs_graph({lp})) {
    auto n = std::make_shared<NllNode>();
    n->targets = t;
    n->in_shape = lp.shape();
    n->reduction = red;
    n->watch_version(t, "targets");
    n->set_inputs({lp});
    attach(out, n);
  }
  return out;
}

// ------------------------------------------------------------------- embedding
namespace {
struct EmbeddingNode : Node {
  Tensor indices;
  Shape w_shape;
  const char* name() const override { return "EmbeddingNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor dw = Tensor::empty(w_shape, g.dtype(), g.device());
    OpCall c;
    c.in[0] = indices;
    c.in[1] = contiguous(g);
    c.out[0] = dw;
    run_kernel(OperatorId::EmbeddingBackward, g.device(), g.dtype(), c);
    return {dw};
  }
  void release_saved() override { indices = Tensor(); }
};
}  // namespace

Tensor embedding(const Tensor& indices, const Tensor& weight) {
  if (weight.ndim() != 2) throw std::invalid_argument("embedding: weight must be 2-D [vocab, dim]");
  if (indices.dtype() != DType::I64 && indices.dtype() != DType::I32)
    throw std::invalid_argument("embedding: indices must be int32 or int64");
  default_dispatcher().check_dtype(OperatorId::Embedding, weight.device(), weight.dtype());
  check_targets_host(indices, weight.shape()[0], "embedding");
  Tensor idx = contiguous(indices);
  if (idx.device() != weight.device()) idx = to(idx, weight.device());
  Shape os = indices.shape();
  os.push_back(weight.shape()[1]);
  Tensor out = Tensor::empty(os, weight.dtype(), weight.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = idx;
    c.in[1] = contiguous(weight.detach());
    c.out[0] = out;
    run_kernel(OperatorId::Embedding, weight.device(), weight.dtype(), c);
  }
  if (needs_graph({weight})) {
    auto n = std::make_shared<EmbeddingNode>();
    n->indices = idx;
    n->w_shape = weight.shape();
    n->watch_version(idx, "indices");
    n->set_inputs({weight});
    attach(out, n);
  }
  return out;
}

// ------------------------------------------------------------------ conv / pool
std::vector<Tensor> conv2d_backward(const Tensor& g, const Tensor& x, const Tensor& w, bool has_bias, int sh, int sw, int ph, int pw,
                                    bool want_dx) {
  Tensor gc = contiguous(g);
  Tensor dx;
  if (want_dx) {
    OpCall ci;
    dx = Tensor::empty(x.shape(), x.dtype(), x.device());
    ci.in[0] = gc; ci.in[1] = w; ci.out[0] = dx;
    ci.i[0] = sh; ci.i[1] = sw; ci.i[2] = ph; ci.i[3] = pw;
    run_kernel(OperatorId::Conv2dBackwardInput, x.device(), x.dtype(), ci);
  }
  OpCall cw;
  Tensor dw = Tensor::empty(w.shape(), w.dtype(), w.device());
  Tensor db;
  if (has_bias) db = Tensor::empty({w.shape()[0]}, w.dtype(), w.device());
  cw.in[0] = gc; cw.in[1] = x; cw.out[0] = dw;
  if (has_bias) cw.out[1] = db;   // a kernel that also reduces the bias gradient fills it and sets i[4]
  cw.i[0] = sh; cw.i[1] = sw; cw.i[2] = ph; cw.i[3] = pw;
  run_kernel(OperatorId::Conv2dBackwardWeight, x.device(), x.dtype(), cw);
  if (has_bias && cw.i[4] == 0) {
    OpCall cb;
    cb.in[0] = gc; cb.out[0] = db;
    run_kernel(OperatorId::Conv2dBackwardBias, x.device(), x.dtype(), cb);
  }
  return {dx, dw, db};
}

namespace {
int64_t conv_extent(int64_t in, int64_t pad, int64_t k, int64_t stride, const char* what) {
  const int64_t padded = in + 2 * pad;
  if (padded < k) throw std::invalid_argument(std::string("conv2d: kernel does not fit the padded ") + what);
  return (padded - k) / stride + 1;
}

struct Conv2dNode : Node {
  Tensor x, w;
  bool has_bias;
  int sh, sw, ph, pw;
  const char* name() const override { return "Conv2DNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    // The input gradient is only computed when something upstream wants it (the first layer of a
    // network usually has an input that does not require grad).
    const bool want_dx = !edges().empty() && edges()[0].kind != GraphEdge::None;
    return conv2d_backward(g, x, w, has_bias, sh, sw, ph, pw, want_dx);
  }
  void release_saved() override { x = Tensor(); w = Tensor(); }
};

struct MaxPoolNode : Node {
  Tensor x;
  int64_t geom[6];
  const char* name() const override { return "MaxPool2DNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor dx = Tensor::empty(x.shape(), x.dtype(), x.device());
    OpCall c;
    c.in[0] = x;
    c.in[1] = contiguous(g);
    c.out[0] = dx;
    for (int i = 0; i < 6; ++i) c.i[i] = geom[i];
    run_kernel(OperatorId::MaxPool2dBackward, x.device(), x.dtype(), c);
    return {dx};
  }
  void release_saved() override { x = Tensor(); }
};
}  // namespace

Tensor conv2d(const Tensor& x, const Tensor& w, const Tensor& b, int sh, int sw, int ph, int pw) {
  check_same_device(x, w, "conv2d");
  check_same_dtype(x, w, "conv2d");
  if (x.ndim() != 4 || w.ndim() != 4) throw std::invalid_argument("conv2d: input and weight must be 4-D (NCHW / OIHW)");
  if (x.shape()[1] != w.shape()[1]) throw std::invalid_argument("conv2d: input channels do not match the weight");
  if (sh < 1 || sw < 1 || ph < 0 || pw < 0) throw std::invalid_argument("conv2d: invalid stride or padding");
  if (b.defined()) {
    check_same_device(x, b, "conv2d");
    check_same_dtype(x, b, "conv2d");
    if (b.ndim() != 1 || b.shape()[0] != w.shape()[0]) throw std::invalid_argument("conv2d: bias must have shape [C_out]");
  }
  default_dispatcher().check_dtype(OperatorId::Conv2d, x.device(), x.dtype());
  const int64_t OH = conv_extent(x.shape()[2], ph, w.shape()[2], sh, "height");
  const int64_t OW = conv_extent(x.shape()[3], pw, w.shape()[3], sw, "width");
  Tensor xc = contiguous(x.detach()), wc = contiguous(w.detach());
  Tensor out = Tensor::empty({x.shape()[0], w.shape()[0], OH, OW}, x.dtype(), x.device());
  if (out.numel()) {
    OpCall c;
    c.in[0] = xc; c.in[1] = wc;
    if (b.defined()) c.in[2] = contiguous(b.detach());
    c.out[0] = out;
    c.i[0] = sh; c.i[1] = sw; c.i[2] = ph; c.i[3] = pw;
    run_kernel(OperatorId::Conv2d, x.device(), x.dtype(), c);
  }
  if (needs_graph({x, w, b})) {
    auto n = std::make_shared<Conv2dNode>();
    n->x = xc; n->w = wc; n->has_bias = b.defined();
    n->sh = sh; n->sw = sw; n->ph = ph; n->pw = pw;
    n->watch_version(x, "input");
    n->watch_version(w, "weight");
    n->set_inputs({x, w, b});
    attach(out, n);
  }
  return out;
}

Tensor maxpool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph, int pw) {
  if (x.ndim() != 4) throw std::invalid_argument("maxpool2d: input must be 4-D (NCHW)");
  if (kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0) throw std::invalid_argument("maxpool2d: invalid geometry");
  if (ph > kh / 2 || pw > kw / 2) throw std::invalid_argument("maxpool2d: padding must be at most half the kernel size");
  default_dispatcher().check_dtype(OperatorId::MaxPool2d, x.device(), x.dtype());
  if (x.shape()[2] + 2 * ph < kh || x.shape()[3] + 2 * pw < kw)
    throw std::invalid_argument("maxpool2d: kernel does not fit the padded input");
  const int64_t OH = (x.shape()[2] + 2 * ph - kh) / sh + 1, OW = (x.shape()[3] + 2 * pw - kw) / sw + 1;
  Tensor xc = contiguous(x.detach());
  Tensor out = Tensor::empty({x.shape()[0], x.shape()[1], OH, OW}, x.dtype(), x.device());
  const int64_t geom[6] = {kh, kw, sh, sw, ph, pw};
  if (out.numel()) {
    OpCall c;
    c.in[0] = xc;
    c.out[0] = out;
    for (int i = 0; i < 6; ++i) c.i[i] = geom[i];
    run_kernel(OperatorId::MaxPool2d, x.device(), x.dtype(), c);
  }
  if (needs_graph({x})) {
    auto n = std::make_shared<MaxPoolNode>();
    n->x = xc;
    for (int i = 0; i < 6; ++i) n->geom[i] = geom[i];
    n->watch_version(x, "input");
    n->set_inputs({x});
    attach(out, n);
  }
  return out;
}

// ------------------------------------------------------------------- LayerNorm
namespace {
struct LayerNormNode : Node {
  Tensor x2, w, mean, rstd;
  bool has_w, has_b;
  Shape x_shape;
  const char* name() const override { return "LayerNormNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const int64_t D = x2.shape()[1];
    Tensor dx = Tensor::empty(x2.shape(), x2.dtype(), x2.device());
    Tensor dw = has_w ? Tensor::empty({D}, x2.dtype(), x2.device()) : Tensor();
    Tensor db = has_b ? Tensor::empty({D}, x2.dtype(), x2.device()) : Tensor();
    OpCall c;
    c.in[0] = x2;
    c.in[1] = w;
    c.in[2] = reshape(contiguous(g), {-1, D});
    c.in[3] = mean;
    c.in[4] = rstd;
    // The gradient that already reached the input along the residual path is added in the same
    // pass (CUDA kernels only; the CPU kernels leave the addition to the engine).
    Tensor addend = offered_addend(0);
    if (addend.defined() && x2.device().is_cuda() && addend.is_contiguous() && addend.numel() == x2.numel() &&
        addend.dtype() == x2.dtype() && addend.device() == x2.device() && reinterpret_cast<uintptr_t>(addend.data()) % 16 == 0) {
      c.in[5] = addend;
      take_addend(0);
    }
    c.out[0] = dx;
    c.out[1] = dw;
    c.out[2] = db;
    run_kernel(OperatorId::LayerNormBackward, x2.device(), x2.dtype(), c);
    return {reshape(dx, x_shape), dw, db};
  }
  void release_saved() override { x2 = Tensor(); w = Tensor(); mean = Tensor(); rstd = Tensor(); }
};
}  // namespace

Tensor layer_norm(const Tensor& x, const Tensor& w, const Tensor& b, double eps) {
  if (x.ndim() < 1 || x.numel() == 0) throw std::invalid_argument("layer_norm: input must be non-empty");
  const int64_t D = x.shape().back();
  for (const Tensor* p : {&w, &b}) {
    if (!p->defined()) continue;
    check_same_device(x, *p, "layer_norm");
    check_same_dtype(x, *p, "layer_norm");
    if (p->ndim() != 1 || p->shape()[0] != D) throw std::invalid_argument("layer_norm: weight/bias must have shape [D]");
  }
  default_dispatcher().check_dtype(OperatorId::LayerNorm, x.device(), x.dtype());
  Tensor x2 = reshape(contiguous(x.detach()), {-1, D});
  const int64_t R = x2.shape()[0];
  Tensor out = Tensor::empty(x.shape(), x.dtype(), x.device());
  Tensor mean = Tensor::empty({R}, DType::F32, x.device()), rstd = Tensor::empty({R}, DType::F32, x.device());
  OpCall c;
  c.in[0] = x2;
  if (w.defined()) c.in[1] = contiguous(w.detach());
  if (b.defined()) c.in[2] = contiguous(b.detach());
  c.out[0] = Tensor::view_of(out, Layout(Shape{R, D}));
  c.out[1] = mean;
  c.out[2] = rstd;
  c.f[0] = eps;
  run_kernel(OperatorId::LayerNorm, x.device(), x.dtype(), c);
  if (needs_graph({x, w, b})) {
    auto n = std::make_shared<LayerNormNode>();
    n->x2 = x2;
    n->w = c.in[1];
    n->mean = mean;
    n->rstd = rstd;
    n->has_w = w.defined();
    n->has_b = b.defined();
    n->x_shape = x.shape();
    n->watch_version(x, "input");
    if (w.defined()) n->watch_version(w, "weight");
    n->set_inputs({x, w, b});
    attach(out, n);
  }
  return out;
}

// ------------------------------------------------------------------- attention
namespace {
struct CausalSoftmaxNode : Node {
  Tensor probs;
  double scale;
  const char* name() const override { return "AttentionSoftmaxNode"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor out = Tensor::empty(probs.shape(), probs.dtype(), probs.device());
    OpCall c;
    c.in[0] = probs;
    c.in[1] = contiguous(g);
    c.out[0] = out;
    c.f[0] = scale;
    run_kernel(OperatorId::CausalSoftmaxBackward, probs.device(), probs.dtype(), c);
    return {out};
  }
  void release_saved() override { probs = Tensor(); }
};

// probs = softmax(scale * scores + mask) with an optional in-kernel causal mask.
Tensor attention_softmax(const Tensor& scores, const Tensor& mask, bool causal, double scale) {
  Tensor sc = contiguous(scores.detach());
  Tensor out = Tensor::empty(scores.shape(), scores.dtype(), scores.device());
  OpCall c;
  c.in[0] = sc;
  if (mask.defined()) c.in[1] = contiguous(mask.detach());
  c.out[0] = out;
  c.f[0] = scale;
  c.i[0] = causal;
  run_kernel(OperatorId::CausalSoftmax, scores.device(), scores.dtype(), c);
  if (needs_graph({scores})) {
    auto n = std::make_shared<CausalSoftmaxNode>();
    n->probs = out.detach();
    n->scale = scale;
    n->watch_version(out, "probabilities");
    n->set_inputs({scores});
    attach(out, n);
  }
  return out;
}
}  // namespace

Tensor attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, bool causal, double scale,
                 double dropout_p, uint64_t seed) {
  check_same_device(q, k, "attention");
  check_same_device(q, v, "attention");
  check_same_dtype(q, k, "attention");
  check_same_dtype(q, v, "attention");
  const int nd = q.ndim();
  if (nd < 3 || nd > 4 || k.ndim() != nd || v.ndim() != nd)
    throw std::invalid_argument("attention: q, k, v must all be 3-D [N, T, D] or 4-D [B, H, T, D]");
  const int64_t Tq = q.shape()[nd - 2], Tk = k.shape()[nd - 2], D = q.shape()[nd - 1];
  if (k.shape()[nd - 1] != D || v.shape()[nd - 2] != Tk) throw std::invalid_argument("attention: q/k/v shape mismatch");
  if (mask.defined()) {
    check_same_device(q, mask, "attention");
    check_same_dtype(q, mask, "attention");
    if (mask.ndim() != 2 || mask.shape()[0] != Tq || mask.shape()[1] != Tk)
      throw std::invalid_argument("attention: mask must have shape [T_q, T_k]");
  }
  Tensor scores = gemm(q, false, k, true);  // [..., Tq, Tk]
  Shape s3{scores.numel() / (Tq * Tk), Tq, Tk};
  Tensor probs = attention_softmax(reshape(scores, s3), mask, causal, scale);
  if (dropout_p > 0.0) probs = dropout(probs, dropout_p, seed);
  return gemm(reshape(probs, scores.shape()), false, v, false);
}

// ------------------------------------------------------------------------ AMP
std::pair<Tensor, bool> amp_unscale_to_f32_and_check(const Tensor& grad, double inv_scale) {
  Tensor out = Tensor::empty(grad.shape(), DType::F32, grad.device());
  if (grad.numel() == 0) return {out, true};
  OpCall c;
  c.in[0] = grad;
  c.out[0] = out;
  c.f[0] = inv_scale;
  run_kernel(OperatorId::AmpUnscale, grad.device(), grad.dtype(), c, layout_of(grad));
  return {out, c.i[0] != 0};
}

Tensor amp_unscale_into(const Tensor& grad, double inv_scale, Tensor& flag) {
  if (flag.dtype() != DType::I32 || flag.numel() != 1 || flag.device() != grad.device())
    throw std::invalid_argument("amp unscale: flag must be a one-element int32 tensor on the gradient's device");
  Tensor out = Tensor::empty(grad.shape(), DType::F32, grad.device());
  if (grad.numel() == 0) return out;
  OpCall c;
  c.in[0] = grad;
  c.in[1] = flag;
  c.out[0] = out;
  c.f[0] = inv_scale;
  run_kernel(OperatorId::AmpUnscale, grad.device(), grad.dtype(), c, layout_of(grad));
  return out;
}

void amp_copy_master_to_model_(Tensor& model, const Tensor& master) {
  if (master.dtype() != DType::F32) throw std::invalid_argument("amp copy: master must be float32");
  if (model.shape() != master.shape()) throw std::invalid_argument("amp copy: shape mismatch");
  check_same_device(model, master, "amp copy");
  if (model.numel()) {
    OpCall c;
    c.in[0] = model;
    c.in[1] = master;
    const bool strided = !model.is_contiguous() || !master.is_contiguous();
    run_kernel(OperatorId::AmpCopy, model.device(), model.dtype(), c, strided ? kStrided : kContiguous);
  }
  model.bump_version();
}

// `stream_kind` 1 queues the update on the device's second (communication) stream; `threads` > 0
// sets the block size (small blocks share an SM with a persistent GEMM CTA of a backward pass).
static void place_update(OpCall& c, const Tensor& master, int stream_kind, int threads) {
  if (threads != 0 && (threads < 32 || threads > 1024 || threads % 32 != 0))
    throw std::invalid_argument("optimizer step: block size must be a multiple of 32 in [32, 1024]");
  c.i[0] = threads;
  if (stream_kind == 1 && master.device().is_cuda()) c.stream = Runtime::instance().cuda(master.device().index).comm_stream();
}

void adam_step_(Tensor& master, Tensor& m, Tensor& v, const Tensor& grad, Tensor& model, const AdamHyper& h, int stream_kind,
                int threads) {
  if (!master.is_contiguous() || !m.is_contiguous() || !v.is_contiguous() || !grad.is_contiguous())
    throw std::invalid_argument("adam_step: tensors must be contiguous");
  if (m.numel() != master.numel() || v.numel() != master.numel() || grad.numel() != master.numel())
    throw std::invalid_argument("adam_step: element counts differ");
  if (master.numel() == 0) return;
  OpCall c;
  c.in[0] = master; c.in[1] = m; c.in[2] = v; c.in[3] = grad;
  if (model.defined()) c.in[4] = model;
  c.f[0] = h.lr; c.f[1] = h.beta1; c.f[2] = h.beta2; c.f[3] = h.eps; c.f[4] = h.weight_decay;
  c.f[5] = h.bias_c1; c.f[6] = h.bias_c2; c.f[7] = h.grad_scale;
  place_update(c, master, stream_kind, threads);
  run_kernel(OperatorId::AdamStep, master.device(), master.dtype(), c);
  master.bump_version(); m.bump_version(); v.bump_version();
  if (model.defined()) model.bump_version();
}

void sgd_step_(Tensor& master, const Tensor& grad, Tensor& model, double lr, double wd, double grad_scale, int stream_kind,
               int threads) {
  if (!master.is_contiguous() || !grad.is_contiguous()) throw std::invalid_argument("sgd_step: tensors must be contiguous");
  if (grad.numel() != master.numel()) throw std::invalid_argument("sgd_step: element counts differ");
  if (master.numel() == 0) return;
  OpCall c;
  c.in[0] = master; c.in[1] = grad;
  if (model.defined()) c.in[2] = model;
  c.f[0] = lr; c.f[1] = wd; c.f[2] = grad_scale;
  place_update(c, master, stream_kind, threads);
  run_kernel(OperatorId::SgdStep, master.device(), master.dtype(), c);
  master.bump_version();
  if (model.defined()) model.bump_version();
}

}  // namespace ops
}  // namespace ob

// ------------------------------------------------- packed-QKV self-attention
namespace ob {
namespace ops {
namespace {

// C = op(A) @ op(B) written into a preallocated (possibly strided) output.
void gemm_out(const Tensor& a, bool ta, const Tensor& b, bool tb, Tensor& out) {
  OpCall c;
  c.in[0] = a;
  c.in[1] = b;
  c.out[0] = out;
  c.i[0] = ta;
  c.i[1] = tb;
  run_kernel(OperatorId::Matmul, a.device(), a.dtype(), c, kStrided);
}

// [B, H, T, dh] view of slot `slot` (0 = q, 1 = k, 2 = v) of a packed [B, T, slots*E] tensor.
Tensor head_view(const Tensor& packed, int slots, int slot, int64_t heads) {
  const int64_t B = packed.shape()[0], T = packed.shape()[1], E = packed.shape()[2] / slots, dh = E / heads;
  const int64_t row = slots * E;
  return Tensor::view_of(packed, Layout(Shape{B, heads, T, dh}, Shape{T * row, dh, row, 1}, packed.offset() + slot * E));
}

Tensor softmax_probs(const Tensor& scores, const Tensor& mask, bool causal, double scale) {
  const int64_t Tq = scores.shape()[2], Tk = scores.shape()[3];
  Tensor out = Tensor::empty(scores.shape(), scores.dtype(), scores.device());
  OpCall c;
  c.in[0] = Tensor::view_of(scores, Layout(Shape{scores.numel() / (Tq * Tk), Tq, Tk}));
  if (mask.defined()) c.in[1] = mask;
  c.out[0] = Tensor::view_of(out, Layout(Shape{scores.numel() / (Tq * Tk), Tq, Tk}));
  c.f[0] = scale;
  c.i[0] = causal;
  run_kernel(OperatorId::CausalSoftmax, scores.device(), scores.dtype(), c);
  return out;
}

struct PackedAttentionNode : Node {
  Tensor qkv, probs, keep;  // keep: dropout mask (scaled) or undefined
  int64_t heads;
  double scale;
  const char* name() const override { return "PackedAttentionNode"; }
  std::vector<Tensor> backward(const Tensor& g_in) override {
    Tensor g = contiguous(g_in);
    Tensor q = head_view(qkv, 3, 0, heads), k = head_view(qkv, 3, 1, heads), v = head_view(qkv, 3, 2, heads);
    Tensor g4 = head_view(g, 1, 0, heads);
    Tensor dqkv = Tensor::empty(qkv.shape(), qkv.dtype(), qkv.device());
    Tensor dq = head_view(dqkv, 3, 0, heads), dk = head_view(dqkv, 3, 1, heads), dv = head_view(dqkv, 3, 2, heads);
    Tensor p_used = keep.defined() ? mul(probs, keep) : probs;
    gemm_out(p_used, true, g4, false, dv);            // dV = Pᵀ dO
    Tensor dp = gemm(g4, false, v, true);              // dP = dO Vᵀ   (no graph: engine runs under no_grad)
    if (keep.defined()) dp = mul(dp, keep);
    Tensor ds = Tensor::empty(probs.shape(), probs.dtype(), probs.device());
    {
      const int64_t Tq = probs.shape()[2], Tk = probs.shape()[3];
      OpCall c;
      c.in[0] = Tensor::view_of(probs, Layout(Shape{probs.numel() / (Tq * Tk), Tq, Tk}));
      c.in[1] = Tensor::view_of(dp, Layout(Shape{probs.numel() / (Tq * Tk), Tq, Tk}));
      c.out[0] = Tensor::view_of(ds, Layout(Shape{probs.numel() / (Tq * Tk), Tq, Tk}));
      c.f[0] = scale;
      run_kernel(OperatorId::CausalSoftmaxBackward, probs.device(), probs.dtype(), c);
    }
    gemm_out(ds, false, k, false, dq);                 // dQ = dS K
    gemm_out(ds, true, q, false, dk);                  // dK = dSᵀ Q
    return {dqkv};
  }
  void release_saved() override { qkv = Tensor(); probs = Tensor(); keep = Tensor(); }
};

// Fused path: the forward keeps only the output and the per-row log-sum-exp; the backward
// recomputes the probabilities tile by tile on the tensor cores.
struct FlashAttentionNode : Node {
  Tensor qkv, out, lse;
  int64_t heads;
  double scale;
  bool causal;
  const char* name() const override { return "FlashAttentionNode"; }
  std::vector<Tensor> backward(const Tensor& g_in) override {
    Tensor g = contiguous(g_in);
    Tensor dqkv = Tensor::empty(qkv.shape(), qkv.dtype(), qkv.device());
    Tensor delta = Tensor::empty(lse.shape(), DType::F32, qkv.device());
    cu::flash_attention_backward_current(qkv, out, lse, g, heads, causal, scale, dqkv, delta);
    return {dqkv};
  }
  void release_saved() override { qkv = Tensor(); out = Tensor(); lse = Tensor(); }
};

}  // namespace

Tensor attention_packed(const Tensor& qkv_in, int64_t heads, const Tensor& mask, bool causal, double scale,
                        double dropout_p, uint64_t seed) {
  if (qkv_in.ndim() != 3 || qkv_in.shape()[2] % 3 != 0)
    throw std::invalid_argument("attention_packed: expected a [B, T, 3*E] tensor");
  const int64_t B = qkv_in.shape()[0], T = qkv_in.shape()[1], E = qkv_in.shape()[2] / 3;
  if (heads < 1 || E % heads != 0) throw std::invalid_argument("attention_packed: E must be divisible by the head count");
  if (mask.defined() && (mask.ndim() != 2 || mask.shape()[0] != T || mask.shape()[1] != T))
    throw std::invalid_argument("attention_packed: mask must have shape [T, T]");
  Tensor qkv = contiguous(qkv_in.detach());
  if (!mask.defined() && dropout_p == 0.0 && cu::flash_attention_supported(qkv, heads)) {
    Tensor out = Tensor::empty({B, T, E}, qkv.dtype(), qkv.device());
    Tensor lse = Tensor::empty({B, heads, T}, DType::F32, qkv.device());
    cu::flash_attention_forward_current(qkv, heads, causal, scale, out, lse);
    if (needs_graph({qkv_in})) {
      auto n = std::make_shared<FlashAttentionNode>();
      n->qkv = qkv;
      n->out = out.detach();
      n->lse = lse;
      n->heads = heads;
      n->scale = scale;
      n->causal = causal;
      n->watch_version(qkv_in, "qkv");
      n->set_inputs({qkv_in});
      attach(out, n);
    }
    return out;
  }
  Tensor q = head_view(qkv, 3, 0, heads), k = head_view(qkv, 3, 1, heads), v = head_view(qkv, 3, 2, heads);
  Tensor scores, probs, keep;
  {
    NoGradGuard ng;
    scores = gemm(q, false, k, true);  // [B, H, T, T]
    probs = softmax_probs(scores, mask.defined() ? contiguous(mask.detach()) : Tensor(), causal, scale);
    if (dropout_p > 0.0) keep = dropout_mask(probs.shape(), dropout_p, seed, probs.dtype(), probs.device());
  }
  Tensor out = Tensor::empty({B, T, E}, qkv.dtype(), qkv.device());
  {
    NoGradGuard ng;
    Tensor out4 = head_view(out, 1, 0, heads);
    Tensor p_used = keep.defined() ? mul(probs, keep) : probs;
    gemm_out(p_used, false, v, false, out4);
  }
  if (needs_graph({qkv_in})) {
    auto n = std::make_shared<PackedAttentionNode>();
    n->qkv = qkv;
    n->probs = probs;
    n->keep = keep;
    n->heads = heads;
    n->scale = scale;
    n->watch_version(qkv_in, "qkv");
    n->set_inputs({qkv_in});
    attach(out, n);
  }
  return out;
}

}  // namespace ops
}  // namespace ob

// KernelRegistry / Dispatcher / schema table.
#include "ob/dispatch.h"

#include <mutex>

namespace ob {

namespace {
constexpr int kOps = static_cast<int>(OperatorId::COUNT);
constexpr int kBackends = static_cast<int>(Backend::COUNT);
constexpr int kDTypes = static_cast<int>(DType::COUNT);
inline size_t slot(OperatorId op, Backend b, DType d) {
  return (static_cast<size_t>(op) * kBackends + static_cast<size_t>(b)) * kDTypes + static_cast<size_t>(d);
}
const char* backend_name(Backend b) { return b == Backend::CPU ? "cpu" : "cuda"; }
}  // namespace

uint8_t layout_of(const Tensor& t) {
  if (t.numel() == 0) return kEmpty;
  return t.is_contiguous() ? kContiguous : kStrided;
}

void KernelRegistry::add_schema(const Schema& s) {
  if (frozen_) throw std::logic_error("registry is frozen");
  const size_t idx = static_cast<size_t>(s.id);
  if (idx >= has_schema_.size()) throw std::logic_error("schema id out of range");
  if (has_schema_[idx]) throw std::logic_error(std::string("duplicate schema id for ") + s.name);
  for (const Schema& o : schemas_)
    if (std::string(o.name) == s.name) throw std::logic_error(std::string("duplicate schema name ") + s.name);
  has_schema_[idx] = true;
  schemas_.push_back(s);
}

const Schema& KernelRegistry::schema(OperatorId op) const {
  for (const Schema& s : schemas_)
    if (s.id == op) return s;
  throw std::logic_error("operator has no schema");
}

void KernelRegistry::add_kernel(OperatorId op, Constraints c, KernelFn fn, const char* name) {
  if (frozen_) throw std::logic_error("registry is frozen");
  const Schema& s = schema(op);
  if (s.composite) throw std::logic_error(std::string("composite operator ") + s.name + " may not own kernels");
  if (fn == nullptr) throw std::logic_error("null kernel");
  for (const KernelRecord& k : kernels_) {
    if (k.op == op && k.constraints.backend == c.backend && (k.constraints.dtypes & c.dtypes) &&
        (k.constraints.layouts & c.layouts))
      throw std::logic_error(std::string("overlapping kernel registration for ") + s.name + " (" + name + " vs " +
                             k.name + ")");
  }
  kernels_.push_back(KernelRecord{op, c, fn, name});
}

void KernelRegistry::expect_kernel(OperatorId op, Backend b, DType d) { expected_.push_back({op, b, d}); }

void KernelRegistry::freeze() {
  table_.assign(static_cast<size_t>(kOps) * kBackends * kDTypes, {});
  for (size_t i = 0; i < kernels_.size(); ++i) {
    const KernelRecord& k = kernels_[i];
    for (int d = 0; d < kDTypes; ++d)
      if (k.constraints.dtypes & (1u << d))
        table_[slot(k.op, k.constraints.backend, static_cast<DType>(d))].push_back(static_cast<int>(i));
  }
  for (const Expect& e : expected_) {
    if (table_[slot(e.op, e.b, e.d)].empty())
      throw std::logic_error(std::string("built-in kernel missing: ") + schema(e.op).name + " " +
                             backend_name(e.b) + " " + dtype_name(e.d));
  }
  frozen_ = true;
}

const KernelRecord* KernelRegistry::find(OperatorId op, Backend b, DType d, uint8_t layout) const {
  if (!frozen_) throw std::logic_error("registry must be frozen before lookup");
  const KernelRecord* hit = nullptr;
  for (int idx : table_[slot(op, b, d)]) {
    const KernelRecord& k = kernels_[idx];
    if (k.constraints.layouts & layout) {
      if (hit) throw std::logic_error(std::string("ambiguous kernel selection for ") + schema(op).name);
      hit = &k;
    }
  }
  return hit;
}

const KernelRecord& Dispatcher::select(const DispatchRequest& r) const {
  const Backend b = backend_of(r.device);
  const KernelRecord* k = reg_.find(r.op, b, r.dtype, r.layout);
  if (!k) {
    const Schema& s = reg_.schema(r.op);
    // Distinguish "dtype unsupported" from "layout unsupported" for clearer errors.
    bool any = false;
    for (uint8_t l : {kContiguous, kStrided, kEmpty})
      if (reg_.find(r.op, b, r.dtype, l)) any = true;
    if (!any)
      throw UnsupportedOperation(std::string(s.name) + ": unsupported dtype " + dtype_name(r.dtype) + " on " +
                                 r.device.str());
    throw UnsupportedOperation(std::string(s.name) + ": unsupported layout for dtype " + dtype_name(r.dtype) +
                               " on " + r.device.str());
  }
  if (k->constraints.capability != Capability::None) {
    if (!r.device.is_cuda()) throw UnsupportedOperation("capability-gated kernel selected for a CPU tensor");
    CudaContext& ctx = Runtime::instance().cuda(r.device.index);
    const bool ok = k->constraints.capability == Capability::Bf16 ? ctx.supports_bf16() : ctx.supports_tcgen05();
    if (!ok)
      throw UnsupportedOperation(std::string(reg_.schema(r.op).name) + ": device " + r.device.str() +
                                 " lacks the capability required by " + k->name);
  }
  if (observer_) observer_(r, *k);
  return *k;
}

void Dispatcher::run(const DispatchRequest& r, OpCall& call) const {
  const KernelRecord& k = select(r);
  if (r.device.is_cuda()) {
    DeviceGuard guard(r.device.index);
    if (!call.stream) call.stream = Runtime::instance().stream_for(r.device);
    k.fn(call);
  } else {
    k.fn(call);
  }
}

void Dispatcher::check_dtype(OperatorId op, Device dev, DType d) const {
  const Backend b = backend_of(dev);
  for (uint8_t l : {kContiguous, kStrided, kEmpty})
    if (reg_.find(op, b, d, l)) return;
  throw UnsupportedOperation(std::string(reg_.schema(op).name) + ": unsupported dtype " + dtype_name(d) + " on " +
                             dev.str());
}

KernelRegistry build_builtin_registry() {
  KernelRegistry r;
#define S(id, name, arity, comp) r.add_schema(Schema{OperatorId::id, name, arity, comp})
  S(Add, "add", 2, false); S(Mul, "mul", 2, false); S(Sub, "sub", 2, true); S(Div, "div", 2, true);
  S(AddInplace, "add_", 2, false); S(MulInplace, "mul_", 1, false);
  S(AddScalar, "add_scalar", 1, false); S(MulScalar, "mul_scalar", 1, false);
  S(Neg, "neg", 1, false); S(Relu, "relu", 1, false); S(Sigmoid, "sigmoid", 1, false); S(Tanh, "tanh", 1, false);
  S(LeakyRelu, "leaky_relu", 1, false); S(Gelu, "gelu", 1, false); S(Exp, "exp", 1, false);
  S(Sqrt, "sqrt", 1, false); S(Reciprocal, "reciprocal", 1, false); S(Log, "log", 1, false);
  S(ReluBackward, "relu_backward", 2, false); S(SigmoidBackward, "sigmoid_backward", 2, false);
  S(TanhBackward, "tanh_backward", 2, false); S(LeakyReluBackward, "leaky_relu_backward", 2, false);
  S(GeluBackward, "gelu_backward", 2, false); S(ExpBackward, "exp_backward", 2, false);
  S(SqrtBackward, "sqrt_backward", 2, false); S(ReciprocalBackward, "reciprocal_backward", 2, false);
  S(Matmul, "matmul", 2, false); S(Linear, "linear", -1, false); S(FusedLinearRelu, "fused_linear_relu", 3, true);
  S(Sum, "sum", 1, false); S(Mean, "mean", 1, false); S(Max, "max", 1, false);
  S(MaxBackward, "max_backward", 2, false); S(Unbroadcast, "unbroadcast", 1, false);
  S(Softmax, "softmax", 1, false); S(SoftmaxBackward, "softmax_backward", 2, false);
  S(LogSoftmax, "log_softmax", 1, false); S(LogSoftmaxBackward, "log_softmax_backward", 2, false);
  S(CrossEntropy, "cross_entropy", 2, false); S(CrossEntropyBackward, "cross_entropy_backward", 3, false);
  S(NllLoss, "nll_loss", 2, false); S(NllLossBackward, "nll_loss_backward", 2, false);
  S(Embedding, "embedding", 2, false); S(EmbeddingBackward, "embedding_backward", 2, false);
  S(DropoutMask, "dropout_mask", 0, false); S(Dropout, "dropout", 1, true);
  S(Conv2d, "conv2d", 3, false); S(Conv2dBackwardInput, "conv2d_backward_input", 2, false);
  S(Conv2dBackwardWeight, "conv2d_backward_weight", 2, false);
  S(Conv2dBackwardBias, "conv2d_backward_bias", 1, false);
  S(MaxPool2d, "maxpool2d", 1, false); S(MaxPool2dBackward, "maxpool2d_backward", 2, false);
  S(LayerNorm, "layer_norm", 3, false); S(LayerNormBackward, "layer_norm_backward", 5, false);
  S(Attention, "attention", -1, false); S(AttentionBackward, "attention_backward", -1, false);
  S(CausalSoftmax, "causal_softmax", 1, false); S(CausalSoftmaxBackward, "causal_softmax_backward", 2, false);
  S(Cast, "cast", 1, false); S(To, "to", 1, false); S(Contiguous, "contiguous", 1, false);
  S(Fill, "fill_", 1, false); S(CopyRange, "copy_range", 2, false); S(ScatterSlice, "scatter_slice", 1, false);
  S(IsFiniteAll, "isfinite_all", 1, false); S(AmpUnscale, "amp_unscale", 1, false); S(AmpCopy, "amp_copy", 2, false);
  S(AdamStep, "adam_step", -1, false); S(SgdStep, "sgd_step", -1, false); S(BiasGrad, "bias_grad", 1, false);
#undef S
  register_cpu_kernels(r);
  register_cuda_kernels(r);
  // Built-ins that must be present in every build.
  for (OperatorId op : {OperatorId::Add, OperatorId::Mul, OperatorId::Matmul, OperatorId::Relu, OperatorId::Sum,
                        OperatorId::CrossEntropy, OperatorId::Contiguous, OperatorId::Cast}) {
    r.expect_kernel(op, Backend::CPU, DType::F32);
    r.expect_kernel(op, Backend::CUDA, DType::F32);
  }
  r.expect_kernel(OperatorId::Matmul, Backend::CUDA, DType::BF16);
  r.expect_kernel(OperatorId::Matmul, Backend::CUDA, DType::F16);
  r.freeze();
  return r;
}

Dispatcher& default_dispatcher() {
  static Dispatcher* d = new Dispatcher(build_builtin_registry());
  return *d;
}

}  // namespace ob

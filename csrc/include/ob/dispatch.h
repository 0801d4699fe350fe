// Operator schema table, frozen kernel registry and dispatcher.
//
// Every backend kernel is registered once as (operator, backend, dtype set, layout
// set, capability) and is looked up through a dense table, so the per-op cost is an
// index computation rather than a scan.  Kernels take a boxed OpCall.
//
// Parity (reference project paths): include/orthon/dispatch/{operator,dispatcher}.h,
// src/dispatch/{kernel_registry,dispatcher,builtin_registration}.cpp.
#pragma once
#include <array>
#include <functional>
#include <string>
#include <vector>

#include "ob/tensor.h"

namespace ob {

enum class OperatorId : uint16_t {
  Add, Mul, Sub, Div, AddInplace, MulInplace, AddScalar, MulScalar,
  Neg, Relu, Sigmoid, Tanh, LeakyRelu, Gelu, Exp, Sqrt, Reciprocal, Log,
  ReluBackward, SigmoidBackward, TanhBackward, LeakyReluBackward, GeluBackward, ExpBackward,
  SqrtBackward, ReciprocalBackward,
  Matmul, Linear, FusedLinearRelu,
  Sum, Mean, Max, MaxBackward, Unbroadcast,
  Softmax, SoftmaxBackward, LogSoftmax, LogSoftmaxBackward,
  CrossEntropy, CrossEntropyBackward, NllLoss, NllLossBackward,
  Embedding, EmbeddingBackward, DropoutMask, Dropout,
  Conv2d, Conv2dBackwardInput, Conv2dBackwardWeight, Conv2dBackwardBias,
  MaxPool2d, MaxPool2dBackward,
  LayerNorm, LayerNormBackward, Attention, AttentionBackward,
  CausalSoftmax, CausalSoftmaxBackward,
  Cast, To, Contiguous, Fill, CopyRange, ScatterSlice,
  IsFiniteAll, AmpUnscale, AmpCopy, AdamStep, SgdStep, BiasGrad,
  COUNT
};

enum class Backend : uint8_t { CPU = 0, CUDA = 1, COUNT };
enum LayoutBit : uint8_t { kContiguous = 1, kStrided = 2, kEmpty = 4 };
enum class Capability : uint8_t { None = 0, Bf16, Tcgen05 };

constexpr uint32_t dtype_bit(DType d) { return 1u << static_cast<int>(d); }
constexpr uint32_t kMaskF32 = dtype_bit(DType::F32);
constexpr uint32_t kMaskF64 = dtype_bit(DType::F64);
constexpr uint32_t kMaskHalf = dtype_bit(DType::F16) | dtype_bit(DType::BF16);
constexpr uint32_t kMaskCpuCompute = kMaskF32 | kMaskF64;
constexpr uint32_t kMaskCudaCompute = kMaskF32 | kMaskHalf;
constexpr uint32_t kMaskAll = (1u << static_cast<int>(DType::COUNT)) - 1;

// Boxed call frame.  Kernels read inputs/attributes and fill preallocated outputs
// (or allocate them when the semantic op left them undefined).
struct OpCall {
  Tensor in[8];
  Tensor out[4];
  double f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t i[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  std::vector<int64_t> list;
  StreamHandle stream = nullptr;
};

using KernelFn = void (*)(OpCall&);

struct Schema {
  OperatorId id;
  const char* name;
  int arity;       // number of tensor inputs the kernel expects (−1: variable)
  bool composite;  // composed from other operators: may not own kernels
};

struct Constraints {
  Backend backend = Backend::CPU;
  uint32_t dtypes = 0;
  uint8_t layouts = kContiguous | kEmpty;
  Capability capability = Capability::None;
};

struct KernelRecord {
  OperatorId op;
  Constraints constraints;
  KernelFn fn;
  const char* name;
};

class UnsupportedOperation : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

class KernelRegistry {
 public:
  void add_schema(const Schema& s);
  void add_kernel(OperatorId op, Constraints c, KernelFn fn, const char* name);
  // Declares that a built-in kernel must exist once the registry is frozen.
  void expect_kernel(OperatorId op, Backend b, DType d);
  void freeze();
  bool frozen() const { return frozen_; }
  const Schema& schema(OperatorId op) const;
  const std::vector<KernelRecord>& kernels() const { return kernels_; }
  // nullptr when nothing matches.
  const KernelRecord* find(OperatorId op, Backend b, DType d, uint8_t layout) const;

 private:
  struct Expect { OperatorId op; Backend b; DType d; };
  std::vector<Schema> schemas_;
  std::vector<bool> has_schema_ = std::vector<bool>(static_cast<size_t>(OperatorId::COUNT), false);
  std::vector<KernelRecord> kernels_;
  std::vector<Expect> expected_;
  // [op][backend][dtype] -> indices into kernels_
  std::vector<std::vector<int>> table_;
  bool frozen_ = false;
};

struct DispatchRequest {
  OperatorId op;
  Device device;
  DType dtype;
  uint8_t layout = kContiguous;
};

class Dispatcher {
 public:
  explicit Dispatcher(KernelRegistry reg) : reg_(std::move(reg)) {}
  const KernelRecord& select(const DispatchRequest& r) const;
  void run(const DispatchRequest& r, OpCall& call) const;
  // Throws UnsupportedOperation when the dtype has no kernel at all on that device.
  void check_dtype(OperatorId op, Device dev, DType d) const;
  const KernelRegistry& registry() const { return reg_; }
  using Observer = std::function<void(const DispatchRequest&, const KernelRecord&)>;
  void set_observer(Observer o) { observer_ = std::move(o); }

 private:
  KernelRegistry reg_;
  Observer observer_;
};

Dispatcher& default_dispatcher();
KernelRegistry build_builtin_registry();
void register_cpu_kernels(KernelRegistry& r);
void register_cuda_kernels(KernelRegistry& r);

inline Backend backend_of(Device d) { return d.is_cuda() ? Backend::CUDA : Backend::CPU; }
uint8_t layout_of(const Tensor& t);

}  // namespace ob

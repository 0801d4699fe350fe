// Semantic operators: validation, dispatch, and graph attachment.
//
// Route of every operator: public op -> validation -> DispatchRequest -> Dispatcher ->
// frozen KernelRegistry -> backend kernel, then a formula Node is attached when any
// input requires grad.  (reference project: docs/architecture.md:51-56, src/ops/*.cpp)
#pragma once
#include <optional>

#include "ob/dispatch.h"
#include "ob/tensor.h"

namespace ob {
namespace ops {

// ---- raw helpers (no graph, no version bump unless stated)
void fill_raw(Tensor& t, double value);
Tensor clone(const Tensor& t);                       // contiguous copy, same device, no graph
void copy_(Tensor& dst, const Tensor& src);          // same shape+dtype; bumps dst version
void copy_range(Tensor& dst, int64_t dst_off, const Tensor& src, int64_t src_off, int64_t n);
double read_scalar(const Tensor& t, int64_t flat_index);
void write_scalar(Tensor& t, int64_t flat_index, double v);

// ---- factories
Tensor zeros_like(const Tensor& t);
Tensor ones_like(const Tensor& t);

// ---- binary / scalar
Tensor add(const Tensor& a, const Tensor& b);
Tensor mul(const Tensor& a, const Tensor& b);
Tensor sub(const Tensor& a, const Tensor& b);
Tensor div(const Tensor& a, const Tensor& b);
Tensor add_scalar(const Tensor& a, double s);
Tensor mul_scalar(const Tensor& a, double s);
Tensor& add_(Tensor& a, const Tensor& b, double alpha);  // a += alpha*b
Tensor& mul_(Tensor& a, double alpha);                   // a *= alpha
Tensor& fill_(Tensor& a, double v);
Tensor unbroadcast(const Tensor& g, const Shape& target);

// ---- unary
enum class Unary : int { Neg, Relu, Sigmoid, Tanh, LeakyRelu, Gelu, Exp, Sqrt, Reciprocal, Log };
Tensor unary(Unary kind, const Tensor& a, double param = 0.0);
Tensor unary_backward(Unary kind, const Tensor& x, const Tensor& grad, double param = 0.0);
inline Tensor neg(const Tensor& a) { return unary(Unary::Neg, a); }
inline Tensor relu(const Tensor& a) { return unary(Unary::Relu, a); }
inline Tensor sigmoid(const Tensor& a) { return unary(Unary::Sigmoid, a); }
inline Tensor tanh(const Tensor& a) { return unary(Unary::Tanh, a); }
inline Tensor leaky_relu(const Tensor& a, double slope) { return unary(Unary::LeakyRelu, a, slope); }
inline Tensor gelu(const Tensor& a) { return unary(Unary::Gelu, a); }
inline Tensor exp(const Tensor& a) { return unary(Unary::Exp, a); }
inline Tensor sqrt(const Tensor& a) { return unary(Unary::Sqrt, a); }
inline Tensor reciprocal(const Tensor& a) { return unary(Unary::Reciprocal, a); }
inline Tensor log(const Tensor& a) { return unary(Unary::Log, a); }
Tensor dropout(const Tensor& a, double p, uint64_t seed);
Tensor dropout_mask(const Shape& shape, double p, uint64_t seed, DType dtype, Device dev);

// ---- shape
Tensor reshape(const Tensor& a, const Shape& shape);
Tensor flatten(const Tensor& a, int start, int end);
Tensor transpose(const Tensor& a, int d0, int d1);
Tensor contiguous(const Tensor& a);
Tensor slice(const Tensor& a, int dim, int64_t start, int64_t end);
Tensor index(const Tensor& a, int64_t i);
Tensor cast(const Tensor& a, DType dtype);
Tensor to(const Tensor& a, Device dev);

// ---- reductions
Tensor sum(const Tensor& a, std::optional<int> dim, bool keepdim);
Tensor mean(const Tensor& a, std::optional<int> dim, bool keepdim);
std::pair<Tensor, Tensor> max(const Tensor& a, std::optional<int> dim, bool keepdim);  // values, int64 indices
Tensor argmax(const Tensor& a, std::optional<int> dim, bool keepdim);
bool isfinite_all(const Tensor& a);
// Sets flag[0] = 1 (int32, same device) when `a` holds a non-finite value; no host sync.
void isfinite_into(const Tensor& a, Tensor& flag);

// ---- linear algebra
Tensor matmul(const Tensor& a, const Tensor& b);
enum class Act : int { None = 0, Relu = 1, Gelu = 2 };
// y = act(x @ w + b) (+ residual).  x [..., in], w [in, out], b [out] or undefined.
Tensor linear(const Tensor& x, const Tensor& w, const Tensor& b, Act act, const Tensor& residual);
Tensor fused_linear_relu(const Tensor& x, const Tensor& w, const Tensor& b);
// gelu(x @ w1 + b1) @ w2 + b2 (+ residual) as one autograd node: the backward multiplies by
// gelu'(pre-activation) inside the epilogue of the input-gradient GEMM.
Tensor mlp_gelu(const Tensor& x, const Tensor& w1, const Tensor& b1, const Tensor& w2, const Tensor& b2, const Tensor& residual);
// Low-level GEMM used by formulas: C = op(A) @ op(B), 2-D or batched 3-D operands.
Tensor gemm(const Tensor& a, bool trans_a, const Tensor& b, bool trans_b);

// ---- nn
Tensor softmax(const Tensor& a, int dim);
Tensor log_softmax(const Tensor& a, int dim);
Tensor cross_entropy(const Tensor& logits, const Tensor& targets);  // mean loss, shape [1]
Tensor cross_entropy_host(const Tensor& logits, const std::vector<int64_t>& targets);
Tensor nll_loss(const Tensor& log_probs, const Tensor& targets, const std::string& reduction);
Tensor embedding(const Tensor& indices, const Tensor& weight);
Tensor conv2d(const Tensor& x, const Tensor& w, const Tensor& b, int sh, int sw, int ph, int pw);
// The three gradients of conv2d for an output gradient g: {dx (undefined unless want_dx), dw, db (undefined unless has_bias)}.
std::vector<Tensor> conv2d_backward(const Tensor& g, const Tensor& x, const Tensor& w, bool has_bias, int sh, int sw, int ph, int pw,
                                    bool want_dx);
Tensor maxpool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph, int pw);
Tensor layer_norm(const Tensor& x, const Tensor& w, const Tensor& b, double eps);
// q,k,v: [B, H, T, D] (any strides with a contiguous last dim).  Additive mask optional
// ([T, T] broadcast over B and H); `causal` applies the lower-triangular mask in-kernel.
Tensor attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, bool causal,
                 double scale, double dropout_p, uint64_t seed);

// Self-attention over a packed projection [B, T, 3*E] (q | k | v along the last dim).  Heads are
// read in place through strided views and the result is written straight into [B, T, E]; the
// backward writes dq/dk/dv into one packed [B, T, 3*E] gradient.  No head transposes are copied.
Tensor attention_packed(const Tensor& qkv, int64_t heads, const Tensor& mask, bool causal, double scale,
                        double dropout_p, uint64_t seed);

// ---- AMP / optimizer kernels
std::pair<Tensor, bool> amp_unscale_to_f32_and_check(const Tensor& grad, double inv_scale);
// Unscales into a new float32 tensor and ORs "saw a non-finite value" into `flag` (int32 [1]
// on the same device) without synchronizing the host.
Tensor amp_unscale_into(const Tensor& grad, double inv_scale, Tensor& flag);
void amp_copy_master_to_model_(Tensor& model, const Tensor& master);
struct AdamHyper {
  double lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
};
// Fused FP32-master Adam over one flat range.  `model` may be undefined or a low-precision
// copy to refresh; `grad` may be F32/F16/BF16.
void adam_step_(Tensor& master, Tensor& m, Tensor& v, const Tensor& grad, Tensor& model, const AdamHyper& h,
                int stream_kind = 0, int threads = 0);
void sgd_step_(Tensor& master, const Tensor& grad, Tensor& model, double lr, double weight_decay,
               double grad_scale, int stream_kind = 0, int threads = 0);

// ---- dispatch glue
void run_kernel(OperatorId op, Device dev, DType dtype, OpCall& call, uint8_t layout = kContiguous);
void check_same_device(const Tensor& a, const Tensor& b, const char* op);
void check_same_dtype(const Tensor& a, const Tensor& b, const char* op);

}  // namespace ops
namespace cu {
// Fused tcgen05 attention over a packed [B, T, 3E] projection (bf16 / f16, head size 64 or 128).
bool flash_attention_supported(const Tensor& qkv, int64_t heads);
void flash_attention_forward_current(const Tensor& qkv, int64_t heads, bool causal, double scale, Tensor& out, Tensor& lse);
void flash_attention_backward_current(const Tensor& qkv, const Tensor& out, const Tensor& lse, const Tensor& dout, int64_t heads,
                                      bool causal, double scale, Tensor& dqkv, Tensor& delta);
}  // namespace cu

}  // namespace ob

// Calling conventions of the boxed backend kernels (OpCall slots per operator).
//
//  Add/Mul            in0=a in1=b out0 (preallocated, broadcast shape); inputs may be strided
//  AddInplace         in0=a (dst) in1=b f0=alpha          a += alpha*b
//  MulInplace         in0=a f0=alpha                      a *= alpha
//  AddScalar/MulScalar in0=a f0=s out0
//  unary              in0=x out0 f0=param
//  unary backward     in0=x in1=grad out0 f0=param
//  Matmul             in0=A in1=B out0=C i0=trans_a i1=trans_b   2-D or batched 3-D
//  Linear             in0=x[M,K] in1=w[K,N] in2=bias? in3=residual? out0=y out1=preact? i0=act
//  Sum/Mean           in0 out0 i0=outer i1=reduce i2=inner
//  Max                in0 out0=values out1=indices(i64) i0..i2
//  MaxBackward        in0=grad in1=indices out0 (zeroed by kernel) i0..i2
//  Unbroadcast        in0=grad out0 list=target shape padded to grad rank
//  Softmax/LogSoftmax in0 out0 i0..i2 ; backward in0=y in1=grad out0 i0..i2
//  CrossEntropy       in0=logits[B,C] in1=targets(i32/i64) out0=loss[1] out1=lse[B] (f32)
//  CrossEntropyBackward in0=logits in1=targets in2=grad[1] in3=lse out0=dlogits
//  NllLoss            in0=logp[N,C] in1=targets out0 i0=reduction(0 none,1 mean,2 sum)
//  NllLossBackward    in0=grad in1=targets out0=dlogp[N,C] i0=reduction
//  Embedding          in0=indices in1=weight[V,D] out0[...,D]
//  EmbeddingBackward  in0=indices in1=grad out0=dW[V,D] (zeroed by kernel)
//  DropoutMask        out0 f0=p i0=seed bits; CUDA only: in0 (optional, packed) -> out0 = in0 * mask
//  Conv2d             in0=x in1=w in2=bias? out0 i0=sh i1=sw i2=ph i3=pw
//  Conv2dBackwardInput  in0=grad in1=w out0=dx i0..i3
//  Conv2dBackwardWeight in0=grad in1=x out0=dw i0..i3
//  Conv2dBackwardBias   in0=grad out0=db
//  MaxPool2d          in0 out0 i0=kh i1=kw i2=sh i3=sw i4=ph i5=pw ; backward in0=x in1=grad out0=dx
//  LayerNorm          in0=x[R,D] in1=w? in2=b? out0=y out1=mean[R] out2=rstd[R] f0=eps
//  LayerNormBackward  in0=x in1=w? in2=grad in3=mean in4=rstd out0=dx out1=dw? out2=db?
//  CausalSoftmax      in0=scores[N,Tq,Tk] in1=mask? out0=probs f0=scale i0=causal
//  CausalSoftmaxBackward in0=probs in1=grad out0=dscores f0=scale
//  Cast               in0 out0 (dispatch dtype = source dtype)
//  To                 in0=src out0=dst (contiguous on the target device)
//  Contiguous         in0=src (any strides) out0=dst (any strides, same shape)
//  Fill               in0=t f0=value
//  CopyRange          in0=dst in1=src i0=dst_off i1=src_off i2=n  (flat, contiguous)
//  IsFiniteAll        in0 -> i0 (1 = all finite)
//  AmpUnscale         in0=grad out0=f32 f0=inv_scale -> i0 (1 = all finite)
//  AmpCopy            in0=model(dst) in1=master(f32 src)
//  AdamStep           in0=master in1=m in2=v in3=grad in4=model? f0=lr f1=b1 f2=b2 f3=eps f4=wd f5=bc1 f6=bc2 f7=grad_scale
//  SgdStep            in0=master in1=grad in2=model? f0=lr f1=wd f2=grad_scale
#pragma once
#include "ob/dispatch.h"

namespace ob {

// Extrema policy shared by both backends: the first logical maximum wins and the first
// NaN beats every number.  (reference project: include/orthon/reduction/extrema.h:7-21)
template <class T>
inline bool extrema_better(T candidate, T best) {
  const bool cn = candidate != candidate, bn = best != best;
  if (bn) return false;
  if (cn) return true;
  return candidate > best;
}

// splitmix64 finalizer used by dropout on both backends; element i of a mask uses the
// top 24 bits of splitmix64(seed + i).  (reference project: src/backends/cpu/unary.cpp:243-267)
inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

}  // namespace ob

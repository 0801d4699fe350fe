// Shared device helpers for the sm_100a kernels: dtype conversion, 16-byte packs,
// warp/block reductions and launch sizing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "ob/kernels.h"

namespace ob {
namespace cu {

template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<double>(double v) { return static_cast<float>(v); }

template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ double from_f<double>(float v) { return v; }

// 16 bytes of T, moved with one 128-bit access.
template <class T>
struct alignas(16) Pack {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <class T>
__device__ __forceinline__ Pack<T> load_pack(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <class T>
__device__ __forceinline__ void store_pack(T* p, const Pack<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `smem` needs 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? smem[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) smem[0] = r;
  }
  __syncthreads();
  return smem[0];
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? smem[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = warp_max(r);
    if (lane == 0) smem[0] = r;
  }
  __syncthreads();
  return smem[0];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride elementwise pass: enough CTAs to fill 148 SMs several times
// over without launching more than the work needs.
inline int ew_grid(int64_t work_items, int threads, int sm_count) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count > 0 ? sm_count : 148) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

// A kernel that is meant to run beside the persistent tcgen05 GEMMs has to live under the same
// shared-memory / L1 split as they do (an SM is configured for one split at a time, and the GEMMs
// ask for the largest shared-memory share): without this hint the driver would pick the smallest
// share for a kernel that uses no shared memory, and its blocks would wait for the GEMM to drain.
template <class Kernel>
inline void prefer_max_shared_carveout(Kernel kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

inline cudaStream_t stream_of(const OpCall& c) { return static_cast<cudaStream_t>(c.stream); }
int sm_count_for(const Tensor& t);
void check_launch(const char* what);

struct Strided {
  int nd;
  int64_t shape[8];
  int64_t st[3][8];
};

}  // namespace cu
}  // namespace ob

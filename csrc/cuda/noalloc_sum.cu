// orthon_sum_f32_noalloc: float32 sum whose block partials live in a static device array, for
// callers that must not allocate.  Declaration and contract: ob/noalloc.h.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "ob/noalloc.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// Block partials of the most recent call.  Every GPU that loads this library holds one copy.
static __device__ __align__(256) float g_noalloc_scratch[ORTHON_NOALLOC_SUM_SCRATCH_FLOATS];

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float smem[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = threadIdx.x < (kThreads >> 5) ? smem[threadIdx.x] : 0.f;
  if (warp == 0) r = warp_sum(r);
  return r;  // valid in thread 0
}

// Block b sums the chunk [b*chunk, min(n, (b+1)*chunk)) and stores one partial.
__global__ void noalloc_partial_kernel(const float* __restrict__ in, long long n, long long chunk,
                                       float* __restrict__ partial) {
  const long long begin = static_cast<long long>(blockIdx.x) * chunk;
  long long end = begin + chunk;
  if (end > n) end = n;
  float acc = 0.f;
  long long i = begin;
  if ((reinterpret_cast<unsigned long long>(in + begin) & 15ull) == 0) {
    const long long nv = (end - begin) / 4;
    const float4* v4 = reinterpret_cast<const float4*>(in + begin);
    for (long long v = threadIdx.x; v < nv; v += kThreads) {
      const float4 x = v4[v];
      acc += (x.x + x.y) + (x.z + x.w);
    }
    i = begin + nv * 4;
  }
  for (long long j = i + threadIdx.x; j < end; j += kThreads) acc += in[j];
  const float total = block_sum(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

// One block adds the partials in index order and writes the result.
__global__ void noalloc_final_kernel(const float* __restrict__ partial, int count, float* __restrict__ out) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += kThreads) acc += partial[i];
  const float total = block_sum(acc);
  if (threadIdx.x == 0) out[0] = total;
}

std::mutex g_setup_mu;
float* g_scratch_addr[kMaxDevices] = {};

void report(char* err, unsigned long cap, const char* text) {
  if (err != nullptr && cap > 0) {
    std::strncpy(err, text, cap - 1);
    err[cap - 1] = '\0';
  }
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int orthon_sum_f32_noalloc(const float* in, long long n, float* out,
                                                                              void* stream, char* err,
                                                                              unsigned long err_cap) {
  if (err != nullptr && err_cap > 0) err[0] = '\0';
  if (out == nullptr || n < 0 || (in == nullptr && n > 0)) {
    report(err, err_cap, "orthon_sum_f32_noalloc: null pointer or negative element count");
    return 1;
  }
  if (n > ORTHON_NOALLOC_SUM_MAX_ELEMENTS) {
    char text[160];
    std::snprintf(text, sizeof(text), "orthon_sum_f32_noalloc: %lld elements exceed the supported maximum of %lld", n,
                  static_cast<long long>(ORTHON_NOALLOC_SUM_MAX_ELEMENTS));
    report(err, err_cap, text);
    return 2;
  }
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess && (device < 0 || device >= kMaxDevices)) e = cudaErrorInvalidDevice;
  float* scratch = nullptr;
  if (e == cudaSuccess) {
    // In host code the array's name is only a handle; the device address has to be asked for,
    // once per device, with that device current.
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_scratch_addr[device] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e == cudaSuccess) g_scratch_addr[device] = static_cast<float*>(p);
    }
    scratch = g_scratch_addr[device];
  }
  if (e == cudaSuccess) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // At least 4096 elements per block, at most one partial per scratch slot.
    long long blocks = (n + 4095) / 4096;
    if (blocks < 1) blocks = 1;
    if (blocks > ORTHON_NOALLOC_SUM_SCRATCH_FLOATS) blocks = ORTHON_NOALLOC_SUM_SCRATCH_FLOATS;
    long long chunk = (n + blocks - 1) / blocks;
    chunk = (chunk + 3) & ~3LL;  // chunk starts stay 16-byte aligned relative to `in`
    if (chunk < 4) chunk = 4;
    blocks = n > 0 ? (n + chunk - 1) / chunk : 1;
    noalloc_partial_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(in, n, chunk, scratch);
    noalloc_final_kernel<<<1, kThreads, 0, st>>>(scratch, static_cast<int>(blocks), out);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    char text[200];
    std::snprintf(text, sizeof(text), "orthon_sum_f32_noalloc: CUDA error: %s", cudaGetErrorString(e));
    report(err, err_cap, text);
    return 3;
  }
  return 0;
}

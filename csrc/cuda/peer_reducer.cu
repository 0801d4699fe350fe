// Peer-memory gradient reducer for one node of NVLink/NVSwitch-connected GPUs.
//
// Every rank maps every other rank's gradient bucket, float32 staging bucket and flag block
// (CUDA IPC, or cuMemCreate allocations shared by file descriptor).  One kernel launch per
// bucket and per rank then does, without any NCCL call or bulk-tensor copy:
//
//   two-shot   entry barrier -> each rank reduces its 1/world slice by reading that slice from
//              every peer (8 / world vectors of every rank in flight per thread), multiplies by
//              `scale` (1/world_size x 1/loss_scale), checks for inf/NaN and writes the result,
//              in the gradient dtype, into that slice of every rank's bucket -> barrier ->
//              every rank applies the FP32-master Adam / SGD update to the whole bucket from
//              its local copy and refreshes the low-precision model copy ("average" mode stops
//              after the barrier).
//   one-shot   entry barrier -> every rank reads the whole bucket from every peer and reduces it
//              into its local float32 staging copy (lowest latency for small buckets) -> barrier
//              (all reads done, inf/NaN verdict known) -> update or write-back from that copy.
//   NVLS       same protocol as two-shot, with the slice reduced by multimem.ld_reduce and
//              re-broadcast by multimem.st through the multicast mapping of the buckets: the
//              NVSwitch adds and replicates, each GPU moves S instead of 2 S (w-1)/w bytes.
//
// Barriers are per-CTA flag words in peer memory written with st.release.sys and polled with
// ld.acquire.sys; CTA b only ever depends on CTA b of the other ranks, and the grid is small
// enough to be co-resident, so no deadlock is possible.  Every poll loop has a time budget (a
// kernel argument, in nanoseconds of the global timer): when it runs out the kernel records an
// error code in a status word and returns, it never traps or spins forever.  Reduction order is
// rank 0..world-1 for every element and each element is reduced by exactly one rank (two-shot),
// so all ranks end up bit-identical.
//
// The entry barrier also carries the participation consensus of the bucket: every rank
// publishes one bit per parameter ("this rank produced a gradient") and an "invalid local
// gradient profile" bit; after the barrier every rank holds the union of the usage bits (read
// by the host only when it needs them) and, if any rank flagged its profile invalid, every rank
// leaves the kernel without touching gradients or parameters and records kErrInvalidProfile.
//
// The block size is a launch parameter: 512 threads when the kernel has the GPU to itself, 128
// when it runs beside the persistent tcgen05 GEMMs of a backward pass, whose CTAs leave about
// 14 K registers per SM free (one 128-thread CTA of this kernel fits, a 512-thread one does not
// and would wait for a GEMM to end and then hold its SM against the next one).
//
// Replaces (reference project paths): the NCCL all-reduce + per-parameter copy/scale path of
// python/orthon/distributed/_reducer.py:61-163, the unscale/inf-check kernels
// src/backends/cuda/unary_kernels.cu:1048-1261, and the composed Adam step
// python/orthon/optim/adam.py:134-183.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <mutex>

#include "ob/cuda_common.cuh"
#include "ob/ops.h"

namespace py = pybind11;

namespace ob {
namespace cu {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 160;
constexpr int kPeerThreads = 512;  // upper bound of the block size
constexpr int kUsageWords = 64;    // one bit per parameter of a bucket: at most 2048 parameters
constexpr uint32_t kInvalidBit = 0x80000000u;

enum : int { kModeAverage = 0, kModeAdam = 1, kModeSgd = 2 };
enum : int { kErrEntryBarrier = 11, kErrMidBarrier = 12, kErrInvalidProfile = 20 };

struct PeerArgs {
  int rank, world, mode, oneshot;
  const void* grads[kMaxRanks];
  float* staging[kMaxRanks];
  uint32_t* flags[kMaxRanks];
  long long n, per;  // elements in the bucket, elements per rank slice (multiple of 8)
  uint32_t epoch;
  float scale;
  float* master;
  float* m;
  float* v;
  void* model;  // same dtype as the gradients, or null
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2;
  const long long* seg_end;  // optional per-parameter weight-decay segments
  const float* seg_wd;
  int nseg;
  void* mc_grads;  // multicast mapping of every rank's bucket (NVLS path), or null
  int* status;     // local: first error code
  int* found_inf;  // local: set to 1 when any rank saw a non-finite reduced gradient
  long long wait_ns;  // budget of every flag wait
  int invalid;        // this rank's gradient profile is invalid: nobody reduces, everybody reports
  int usage_words;    // number of valid words in `usage`
  uint32_t usage[kUsageWords];  // bit i of word w: parameter 32 w + i of the bucket has a local gradient
};

// Flag block layout (uint32 words): [phase 0..2][cta][src rank], one found-inf word (padded to
// 8), the usage words of every source rank, and the union of them (local result).
__host__ __device__ inline size_t flag_words() { return 3 * kMaxCtas * kMaxRanks + 8 + (kMaxRanks + 1) * kUsageWords; }
__device__ __forceinline__ uint32_t* flag_at(uint32_t* base, int phase, int cta, int src) {
  return base + (static_cast<size_t>(phase) * kMaxCtas + cta) * kMaxRanks + src;
}
__device__ __forceinline__ uint32_t* inf_word(uint32_t* base) { return base + 3 * kMaxCtas * kMaxRanks; }
__host__ __device__ inline size_t usage_offset(int src) { return 3 * kMaxCtas * kMaxRanks + 8 + static_cast<size_t>(src) * kUsageWords; }
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs with the same index on all ranks meet here.  Returns 0 after a timeout, 2 when a
// rank tagged its arrival with the invalid-profile bit, 1 otherwise.  The low 31 bits of a flag
// word are the epoch of the launch it belongs to.
__device__ int peer_barrier(const PeerArgs& a, int phase, int err_code, uint32_t tag = 0) {
  __syncthreads();
  int ok = 1, tagged = 0;
  if (threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(flag_at(a.flags[threadIdx.x], phase, blockIdx.x, a.rank), a.epoch | tag);
    const uint32_t* mine = flag_at(a.flags[a.rank], phase, blockIdx.x, threadIdx.x);
    const long long t0 = global_ns();
    uint32_t seen;
    while (((seen = ld_acquire_sys(mine)) & ~kInvalidBit) != a.epoch) {
      if (global_ns() - t0 > a.wait_ns) {
        atomicCAS(a.status, 0, err_code);
        ok = 0;
        break;
      }
    }
    tagged = ok && (seen & kInvalidBit) != 0;
  }
  const int any_tag = __syncthreads_or(tagged);
  if (!__syncthreads_and(ok)) return 0;
  return any_tag ? 2 : 1;
}

// Entry of every variant: publish this rank's usage bits (CTA 0), meet the peers, collect the
// union of the usage bits, and agree on the validity of the step.  Returns false when the kernel
// has to leave (timeout, or some rank's gradient profile is invalid).
__device__ bool peer_entry(const PeerArgs& a) {
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < a.usage_words) {
    for (int s = 0; s < a.world; ++s) a.flags[s][usage_offset(a.rank) + threadIdx.x] = a.usage[threadIdx.x];
  }
  const int r = peer_barrier(a, 0, kErrEntryBarrier, a.invalid ? kInvalidBit : 0u);
  if (r == 0) return false;
  if (r == 2) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, kErrInvalidProfile);
    return false;
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < a.usage_words) {
    uint32_t u = 0;
    for (int s = 0; s < a.world; ++s) u |= a.flags[a.rank][usage_offset(s) + threadIdx.x];
    a.flags[a.rank][usage_offset(kMaxRanks) + threadIdx.x] = u;
  }
  return true;
}

// Publishes "this CTA saw a non-finite reduced gradient" to every rank, meets the peers and
// returns whether CTA `blockIdx.x` of any rank did (-1 after a timeout).  Every CTA that learns
// of a non-finite value raises the host-visible flag itself: CTA b only sees the words written by
// CTA b of the other ranks before its barrier, so the union over a rank's CTAs is what makes the
// host flag complete and identical on every rank.
__device__ int exchange_found_inf(const PeerArgs& a, bool bad) {
  const int cta_bad = __syncthreads_or(bad ? 1 : 0);
  if (cta_bad && threadIdx.x < a.world) *inf_word(a.flags[threadIdx.x]) = a.epoch;  // tell every rank
  if (!peer_barrier(a, 1, kErrMidBarrier)) return -1;
  const bool any_inf = ld_acquire_sys(inf_word(a.flags[a.rank])) == a.epoch;
  if (any_inf && threadIdx.x == 0) atomicExch(a.found_inf, 1);
  return any_inf ? 1 : 0;
}

__device__ __forceinline__ float decay_for(const PeerArgs& a, long long e) {
  if (a.nseg == 0) return a.wd;
  int lo = 0, hi = a.nseg - 1;  // first segment whose end is > e
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a.seg_end[mid] > e) hi = mid; else lo = mid + 1;
  }
  return a.seg_wd[lo];
}

// Applies the optimizer to VEC consecutive elements starting at `e` with reduced gradients g[].
template <class GT, int VEC>
__device__ __forceinline__ void apply_update(const PeerArgs& a, long long e, const float* g) {
  const float wd = decay_for(a, e);
  float p[VEC];
#pragma unroll
  for (int k = 0; k < VEC; k += 4) *reinterpret_cast<float4*>(p + k) = *reinterpret_cast<const float4*>(a.master + e + k);
  if (a.mode == kModeAdam) {
    float mm[VEC], vv[VEC];
#pragma unroll
    for (int k = 0; k < VEC; k += 4) {
      *reinterpret_cast<float4*>(mm + k) = *reinterpret_cast<const float4*>(a.m + e + k);
      *reinterpret_cast<float4*>(vv + k) = *reinterpret_cast<const float4*>(a.v + e + k);
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float mi = mm[k], vi = vv[k], w = p[k];
      mi = mi + (a.b1 - 1.f) * mi;
      mi = mi + (1.f - a.b1) * g[k];
      vi = vi + (a.b2 - 1.f) * vi;
      vi = vi + (1.f - a.b2) * (g[k] * g[k]);
      const float denom = sqrtf(vi * a.inv_bc2) + a.eps;
      if (wd != 0.f) w = w + (-a.lr * wd) * w;
      w = w + (-a.lr * a.inv_bc1) * (mi / denom);
      mm[k] = mi; vv[k] = vi; p[k] = w;
    }
#pragma unroll
    for (int k = 0; k < VEC; k += 4) {
      *reinterpret_cast<float4*>(a.m + e + k) = *reinterpret_cast<float4*>(mm + k);
      *reinterpret_cast<float4*>(a.v + e + k) = *reinterpret_cast<float4*>(vv + k);
    }
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float w = p[k];
      if (wd != 0.f) w = w + (-a.lr * wd) * w;
      p[k] = w + (-a.lr) * g[k];
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; k += 4) *reinterpret_cast<float4*>(a.master + e + k) = *reinterpret_cast<float4*>(p + k);
  if (a.model != nullptr) {
    Pack<GT> out;
#pragma unroll
    for (int k = 0; k < VEC; ++k) out.v[k] = from_f<GT>(p[k]);
    store_pack(static_cast<GT*>(a.model) + e, out);
  }
}

// Number of ranks known at compile time (W = 2, 4, 8) lets one thread keep U = 8 / W vectors
// of every rank in flight, so the NVLink round trip is covered at any world size; W = 0 is the
// generic fallback (runtime world, one vector at a time).
template <int W>
struct Unroll {
  static constexpr int kRanks = W ? W : kMaxRanks;
  static constexpr int kVectors = W ? 8 / W : 1;
};

// Scales VEC summed elements, reports non-finite values.
template <int VEC>
__device__ __forceinline__ bool finish_sum(const PeerArgs& a, float* acc) {
  bool bad = false;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    acc[k] *= a.scale;
    bad |= !isfinite(acc[k]);
  }
  return bad;
}

// Reduces the vectors [0, nvec) of the slice starting at element `lo` over all ranks (fixed
// rank order, fp32 accumulation) and hands every reduced vector to `emit(element, acc)`.
template <class GT, int W, class Emit>
__device__ __forceinline__ bool reduce_range(const PeerArgs& a, long long lo, long long nvec, Emit emit) {
  constexpr int VEC = Pack<GT>::N;
  constexpr int R = Unroll<W>::kRanks, U = Unroll<W>::kVectors;
  const int world = W ? W : a.world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  bool bad = false;
  for (long long v0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * U) {
    Pack<GT> in[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vi = v0 + u * stride;
      if (vi < nvec) {
#pragma unroll
        for (int s = 0; s < R; ++s)
          if (s < world) in[u][s] = load_pack(static_cast<const GT*>(a.grads[s]) + lo + vi * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vi = v0 + u * stride;
      if (vi < nvec) {
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
#pragma unroll
        for (int s = 0; s < R; ++s)
          if (s < world) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] += to_f(in[u][s].v[k]);
          }
        bad |= finish_sum<VEC>(a, acc);
        emit(lo + vi * VEC, acc);
      }
    }
  }
  return bad;
}

// Optimizer update from the reduced gradients in the local bucket (two-shot and NVLS variants).
// CTA b consumes, in every slice, exactly the vectors CTA b of the slice's owner produced: the
// barrier between the phases only pairs CTAs of the same index.
template <class GT>
__device__ __forceinline__ void update_from_bucket(const PeerArgs& a) {
  constexpr int VEC = Pack<GT>::N;
  const GT* red = static_cast<const GT*>(a.grads[a.rank]);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int s = 0; s < a.world; ++s) {
    const long long lo = min(a.n, static_cast<long long>(s) * a.per), hi = min(a.n, lo + a.per);
    const long long nvec = (hi - lo) / VEC;
    for (long long vi = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; vi < nvec; vi += stride) {
      const long long e = lo + vi * VEC;
      const Pack<GT> in = load_pack(red + e);
      float g[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) g[k] = to_f(in.v[k]);
      apply_update<GT, VEC>(a, e, g);
    }
  }
}

template <class GT, int W>
__global__ void __launch_bounds__(kPeerThreads) peer_reduce_kernel(PeerArgs a) {
  constexpr int VEC = Pack<GT>::N;  // 16 bytes of gradients per access
  constexpr int R = Unroll<W>::kRanks;
  const int world = W ? W : a.world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (!peer_entry(a)) return;

  bool bad = false;
  if (a.oneshot) {
    // Every rank reduces everything; the update (or write-back) follows immediately.
    bad = reduce_range<GT, W>(a, 0, a.n / VEC, [&](long long e, const float* acc) {
#pragma unroll
      for (int k = 0; k < VEC; k += 4)
        *reinterpret_cast<float4*>(a.staging[a.rank] + e + k) = *reinterpret_cast<const float4*>(acc + k);
    });
  } else {
    const long long lo = min(a.n, static_cast<long long>(a.rank) * a.per), hi = min(a.n, lo + a.per);
    // The reduced slice goes straight back into every rank's bucket in the gradient dtype (no
    // other rank reads this slice); a fused optimizer then reads the local bucket.
    bad = reduce_range<GT, W>(a, lo, (hi - lo) / VEC, [&](long long e, const float* acc) {
      Pack<GT> out;
#pragma unroll
      for (int k = 0; k < VEC; ++k) out.v[k] = from_f<GT>(acc[k]);
#pragma unroll
      for (int s = 0; s < R; ++s)
        if (s < world) store_pack(const_cast<GT*>(static_cast<const GT*>(a.grads[s])) + e, out);
    });
  }
  if (exchange_found_inf(a, bad) < 0) return;

  if (a.oneshot && a.mode == kModeAverage) {
    // The barrier above doubles as "every peer has finished reading this rank's bucket", so
    // the locally staged averages can now overwrite it.
    const long long nvec = a.n / VEC;
    GT* mine = const_cast<GT*>(static_cast<const GT*>(a.grads[a.rank]));
    for (long long vi = first; vi < nvec; vi += stride) {
      Pack<GT> out;
#pragma unroll
      for (int k = 0; k < VEC; ++k) out.v[k] = from_f<GT>(a.staging[a.rank][vi * VEC + k]);
      store_pack(mine + vi * VEC, out);
    }
    return;
  }

  // Fused optimizer: applied to whatever was reduced, like an optimizer step that follows an
  // all-reduce without a loss scaler.  A step that must be skipped on overflow (GradScaler) runs
  // in average mode and applies the update after the host has read the verdict.
  if (a.mode != kModeAverage) {
    const float* red = a.staging[a.rank];
    if (a.oneshot) {
      const long long nvec = a.n / VEC;
      for (long long vi = first; vi < nvec; vi += stride) {
        float g[VEC];
#pragma unroll
        for (int k = 0; k < VEC; k += 4) *reinterpret_cast<float4*>(g + k) = *reinterpret_cast<const float4*>(red + vi * VEC + k);
        apply_update<GT, VEC>(a, vi * VEC, g);
      }
    } else {
      update_from_bucket<GT>(a);
    }
  }
}

// ------------------------------------------------------------------ NVLS path
// multimem.ld_reduce sums one 16-byte vector over every rank's bucket inside the NVSwitch
// (fp32 accumulation for 16-bit gradients) and multimem.st writes the result to every rank at
// once, so each GPU moves S bytes per direction instead of 2 S (w-1)/w.
template <class GT>
__device__ __forceinline__ void multimem_ld_reduce(const void* mc, uint32_t (&r)[4]);
template <>
__device__ __forceinline__ void multimem_ld_reduce<float>(const void* mc, uint32_t (&r)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(mc) : "memory");
}
template <>
__device__ __forceinline__ void multimem_ld_reduce<__nv_bfloat16>(const void* mc, uint32_t (&r)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(mc) : "memory");
}
template <>
__device__ __forceinline__ void multimem_ld_reduce<__half>(const void* mc, uint32_t (&r)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(mc) : "memory");
}
__device__ __forceinline__ void multimem_st(void* mc, const uint32_t (&r)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}

// Same protocol as peer_reduce_kernel (entry barrier, reduce own slice, found-inf word, middle
// barrier, optimizer update on the local copy), with the slice reduced and re-broadcast in the
// switch.  The reduced gradients land in every rank's bucket in the gradient dtype; the update
// reads them from the local bucket.
template <class GT>
__global__ void __launch_bounds__(kPeerThreads) nvls_reduce_kernel(PeerArgs a) {
  constexpr int VEC = Pack<GT>::N;
  constexpr int U = 4;  // vectors in flight per thread
  if (!peer_entry(a)) return;

  const long long lo = min(a.n, static_cast<long long>(a.rank) * a.per), hi = min(a.n, lo + a.per);
  const long long nvec = (hi - lo) / VEC;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  GT* mc = static_cast<GT*>(a.mc_grads);
  bool bad = false;
  for (long long v0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * U) {
    uint32_t raw[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vi = v0 + u * stride;
      if (vi < nvec) multimem_ld_reduce<GT>(mc + lo + vi * VEC, raw[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vi = v0 + u * stride;
      if (vi < nvec) {
        Pack<GT> in = *reinterpret_cast<Pack<GT>*>(raw[u]);
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = to_f(in.v[k]);
        bad |= finish_sum<VEC>(a, acc);
        Pack<GT> out;
#pragma unroll
        for (int k = 0; k < VEC; ++k) out.v[k] = from_f<GT>(acc[k]);
        multimem_st(mc + lo + vi * VEC, *reinterpret_cast<uint32_t(*)[4]>(&out));
      }
    }
  }
  if (exchange_found_inf(a, bad) < 0) return;
  if (a.mode != kModeAverage) update_from_bucket<GT>(a);
}

__global__ void peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
}

struct PeerAllocation {
  void* ptr;
  int device;
  bool opened;
};
std::mutex g_peer_mu;
std::vector<PeerAllocation> g_peer_allocs;

cudaStream_t pick_stream(int device, int kind) {
  CudaContext& ctx = Runtime::instance().cuda(device);
  return static_cast<cudaStream_t>(kind == 1 ? ctx.comm_stream() : ctx.current_stream());
}

}  // namespace
}  // namespace cu

void bind_peer(py::module_& m) {
  using namespace cu;
  m.attr("_PEER_FLAG_BYTES") = py::int_(flag_words() * sizeof(uint32_t));
  m.attr("_PEER_MAX_RANKS") = py::int_(kMaxRanks);

  // Device memory that other processes on this node can map.  Zero-initialised.
  m.def("_peer_alloc", [](size_t bytes, int device) {
    DeviceGuard g(device);
    void* p = nullptr;
    OB_CUDA(cudaMalloc(&p, bytes));
    OB_CUDA(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    OB_CUDA(cudaIpcGetMemHandle(&h, p));
    {
      std::lock_guard<std::mutex> lock(g_peer_mu);
      g_peer_allocs.push_back({p, device, false});
    }
    return py::make_tuple(reinterpret_cast<uintptr_t>(p), py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
  });
  m.def("_peer_open", [](const py::bytes& handle, int device) {
    const std::string s = handle;
    if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("peer handle has the wrong size");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, s.data(), sizeof(h));
    DeviceGuard g(device);
    void* p = nullptr;
    OB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    {
      std::lock_guard<std::mutex> lock(g_peer_mu);
      g_peer_allocs.push_back({p, device, true});
    }
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("_peer_release_all", [] {
    std::lock_guard<std::mutex> lock(g_peer_mu);
    for (auto it = g_peer_allocs.rbegin(); it != g_peer_allocs.rend(); ++it) {
      cudaSetDevice(it->device);
      if (it->opened) cudaIpcCloseMemHandle(it->ptr);
    }
    for (auto& a : g_peer_allocs) {
      if (!a.opened) { cudaSetDevice(a.device); cudaFree(a.ptr); }
    }
    g_peer_allocs.clear();
  });
  // Same-process peers (tests on one box with one process): plain peer access.
  m.def("_peer_enable_access", [](int device, int peer) {
    DeviceGuard g(device);
    int can = 0;
    OB_CUDA(cudaDeviceCanAccessPeer(&can, device, peer));
    if (!can) return false;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) OB_CUDA(e);
    cudaGetLastError();
    return true;
  });
  m.def("_tensor_from_ptr", [](uintptr_t ptr, const std::vector<int64_t>& shape, const std::string& dtype, int device) {
    const DType d = parse_dtype(dtype);
    const size_t bytes = static_cast<size_t>(Layout::checked_numel(shape)) * dtype_size(d);
    auto buf = std::make_shared<Buffer>(Allocation::external(reinterpret_cast<void*>(ptr), bytes, Device(DeviceType::CUDA, device), nullptr));
    return Tensor(std::make_shared<TensorImpl>(buf, Layout(shape), d));
  });
  // Orders stream `dst` after everything queued so far on stream `src` (0 = compute, 1 = comm, 2 = copy).
  m.def("_stream_fence", [](int device, int src, int dst) {
    CudaContext& ctx = Runtime::instance().cuda(device);
    auto pick = [&](int k) { return k == 1 ? ctx.comm_stream() : (k == 2 ? ctx.copy_stream() : ctx.compute_stream()); };
    DeviceGuard g(device);
    CompletionToken t = CompletionToken::record_on(device, pick(src));
    t.enqueue_wait_on(pick(dst));
  });
  m.def("_peer_copy", [](uintptr_t dst, uintptr_t src, size_t bytes, int device, int stream_kind) {
    if (bytes % 16 != 0 || (dst & 15u) || (src & 15u)) throw std::invalid_argument("_peer_copy: 16-byte alignment required");
    DeviceGuard g(device);
    const long long n16 = static_cast<long long>(bytes / 16);
    peer_copy_kernel<<<ew_grid(n16, 256, Runtime::instance().cuda(device).sm_count()), 256, 0, pick_stream(device, stream_kind)>>>(
        reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), n16);
    check_launch("peer copy");
  });
  m.def("_peer_reduce", [](int rank, int world, int device, const std::vector<uintptr_t>& grads, const std::vector<uintptr_t>& staging,
                           const std::vector<uintptr_t>& flags, long long n, const std::string& dtype, uint32_t epoch, double scale,
                           const std::string& mode, bool oneshot, const py::object& master, const py::object& mom, const py::object& var,
                           const py::object& model, const py::dict& hyper, Tensor& status, Tensor& found_inf, int ctas, int stream_kind,
                           uintptr_t mc_grads, int threads, double wait_ms, bool invalid, const std::vector<uint32_t>& usage) {
    if (world < 1 || world > kMaxRanks) throw std::invalid_argument("peer reduce supports 1..8 ranks");
    if (static_cast<int>(grads.size()) != world || static_cast<int>(staging.size()) != world || static_cast<int>(flags.size()) != world)
      throw std::invalid_argument("peer reduce: one gradient, staging and flag pointer per rank is required");
    if (n % 8 != 0) throw std::invalid_argument("peer reduce: bucket length must be a multiple of 8 elements");
    if (threads < 32 || threads > kPeerThreads || threads % 32 != 0) throw std::invalid_argument("peer reduce: block size must be a multiple of 32 in [32, 512]");
    if (usage.size() > static_cast<size_t>(kUsageWords)) throw std::invalid_argument("peer reduce: at most 2048 parameters per bucket");
    if (!(wait_ms > 0.0)) throw std::invalid_argument("peer reduce: the wait budget must be positive");
    PeerArgs a{};
    a.wait_ns = static_cast<long long>(wait_ms * 1e6);
    a.invalid = invalid ? 1 : 0;
    a.usage_words = static_cast<int>(usage.size());
    for (size_t i = 0; i < usage.size(); ++i) a.usage[i] = usage[i];
    a.rank = rank; a.world = world; a.oneshot = oneshot ? 1 : 0;
    a.mode = mode == "adam" ? kModeAdam : (mode == "sgd" ? kModeSgd : kModeAverage);
    if (a.mode == kModeAverage && mode != "average") throw std::invalid_argument("peer reduce: mode must be average, adam or sgd");
    for (int s = 0; s < world; ++s) {
      a.grads[s] = reinterpret_cast<const void*>(grads[s]);
      a.staging[s] = reinterpret_cast<float*>(staging[s]);
      a.flags[s] = reinterpret_cast<uint32_t*>(flags[s]);
    }
    a.mc_grads = reinterpret_cast<void*>(mc_grads);
    a.n = n;
    a.per = (((n + world - 1) / world) + 7) & ~7LL;
    a.epoch = epoch;
    a.scale = static_cast<float>(scale);
    const DType gd = parse_dtype(dtype);
    if (a.mode != kModeAverage) {
      Tensor mt = master.cast<Tensor>();
      if (mt.dtype() != DType::F32 || mt.numel() != n || !mt.is_contiguous()) throw std::invalid_argument("peer reduce: master must be contiguous float32 of the bucket length");
      a.master = mt.data_as<float>();
      if (a.mode == kModeAdam) {
        Tensor m1 = mom.cast<Tensor>(), v1 = var.cast<Tensor>();
        if (m1.numel() != n || v1.numel() != n || m1.dtype() != DType::F32 || v1.dtype() != DType::F32) throw std::invalid_argument("peer reduce: Adam moments must be float32 of the bucket length");
        a.m = m1.data_as<float>();
        a.v = v1.data_as<float>();
      }
      if (!model.is_none()) {
        Tensor md = model.cast<Tensor>();
        if (md.dtype() != gd || md.numel() != n) throw std::invalid_argument("peer reduce: model copy must match the gradient dtype and bucket length");
        a.model = md.data();
      }
      auto f = [&](const char* k, double dflt) { return hyper.contains(k) ? hyper[k].cast<double>() : dflt; };
      a.lr = static_cast<float>(f("lr", 0.0)); a.b1 = static_cast<float>(f("beta1", 0.9)); a.b2 = static_cast<float>(f("beta2", 0.999));
      a.eps = static_cast<float>(f("eps", 1e-8)); a.wd = static_cast<float>(f("weight_decay", 0.0));
      a.inv_bc1 = static_cast<float>(1.0 / f("bias_c1", 1.0)); a.inv_bc2 = static_cast<float>(1.0 / f("bias_c2", 1.0));
      if (hyper.contains("seg_end")) {
        Tensor se = hyper["seg_end"].cast<Tensor>(), sw = hyper["seg_wd"].cast<Tensor>();
        a.seg_end = se.data_as<long long>(); a.seg_wd = sw.data_as<float>(); a.nseg = static_cast<int>(se.numel());
      }
    }
    a.status = status.data_as<int>();
    a.found_inf = found_inf.data_as<int>();
    DeviceGuard g(device);
    const int sms = Runtime::instance().cuda(device).sm_count();
    // Large buckets are bandwidth-bound in the update phase and want every SM; small ones want
    // few CTAs so the flag exchange stays cheap.
    int grid = ctas > 0 ? ctas : std::max(8, std::min(kMaxCtas, (n >= (8ll << 20)) ? sms : sms / 2));
    const long long vecs = n / (gd == DType::F32 ? 4 : 8);
    grid = static_cast<int>(std::max<long long>(1, std::min<long long>(grid, (vecs / world + threads - 1) / threads)));
    if (grid > kMaxCtas) grid = kMaxCtas;
    cudaStream_t st = pick_stream(device, stream_kind);
#define OB_PEER_LAUNCH_W(GT, W)                                                                 \
  do {                                                                                         \
    static const bool once = (prefer_max_shared_carveout(peer_reduce_kernel<GT, W>), true);    \
    (void)once;                                                                                \
    peer_reduce_kernel<GT, W><<<grid, threads, 0, st>>>(a);                                    \
  } while (0)
#define OB_PEER_LAUNCH(GT)                        \
  do {                                            \
    if (world == 2) OB_PEER_LAUNCH_W(GT, 2);      \
    else if (world == 4) OB_PEER_LAUNCH_W(GT, 4); \
    else if (world == 8) OB_PEER_LAUNCH_W(GT, 8); \
    else OB_PEER_LAUNCH_W(GT, 0);                 \
  } while (0)
    if (mc_grads != 0) {
      // In-switch reduction and broadcast through the multicast mapping of the bucket.
      static const bool once = (prefer_max_shared_carveout(nvls_reduce_kernel<float>), prefer_max_shared_carveout(nvls_reduce_kernel<__nv_bfloat16>),
                                prefer_max_shared_carveout(nvls_reduce_kernel<__half>), true);
      (void)once;
      if (gd == DType::F32) nvls_reduce_kernel<float><<<grid, threads, 0, st>>>(a);
      else if (gd == DType::BF16) nvls_reduce_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(a);
      else if (gd == DType::F16) nvls_reduce_kernel<__half><<<grid, threads, 0, st>>>(a);
      else throw std::invalid_argument("peer reduce: gradients must be float32, float16 or bfloat16");
    } else if (gd == DType::F32) OB_PEER_LAUNCH(float);
    else if (gd == DType::BF16) OB_PEER_LAUNCH(__nv_bfloat16);
    else if (gd == DType::F16) OB_PEER_LAUNCH(__half);
    else throw std::invalid_argument("peer reduce: gradients must be float32, float16 or bfloat16");
#undef OB_PEER_LAUNCH
#undef OB_PEER_LAUNCH_W
    check_launch("peer reduce");
    return grid;
  }, py::arg("rank"), py::arg("world"), py::arg("device"), py::arg("grads"), py::arg("staging"), py::arg("flags"), py::arg("n"),
     py::arg("dtype"), py::arg("epoch"), py::arg("scale"), py::arg("mode"), py::arg("oneshot"), py::arg("master") = py::none(),
     py::arg("m") = py::none(), py::arg("v") = py::none(), py::arg("model") = py::none(), py::arg("hyper") = py::dict(),
     py::arg("status"), py::arg("found_inf"), py::arg("ctas") = 0, py::arg("stream_kind") = 1, py::arg("mc_grads") = 0,
     py::arg("threads") = kPeerThreads, py::arg("wait_ms") = 2000.0, py::arg("invalid") = false,
     py::arg("usage") = std::vector<uint32_t>());
  m.attr("_PEER_USAGE_WORD_OFFSET") = py::int_(usage_offset(kMaxRanks));
  m.attr("_PEER_USAGE_WORDS") = py::int_(kUsageWords);
  m.attr("_PEER_ERR_INVALID_PROFILE") = py::int_(static_cast<int>(kErrInvalidProfile));
}

}  // namespace ob

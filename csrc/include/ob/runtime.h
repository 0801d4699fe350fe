// Execution contexts, streams, completion tokens and the caching memory pool.
//
// One CudaContext per device ordinal owns three non-blocking streams (compute,
// communication, copy) and the device facts kernels size their grids from.  The
// MemoryPool is stream-ordered: a block freed and re-acquired on the same stream
// needs no wait; blocks that were touched by another stream carry completion
// events that must have fired before the block is handed out again.
//
// Parity (reference project paths): src/runtime/{runtime,cuda_context,cuda_stream,
// completion}.cpp, src/memory/{pool,allocation,allocator,scratch,raw_allocator}.cpp,
// include/orthon/runtime/cuda_resources.h:18-38 (injectable seam).
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "ob/core.h"

namespace ob {

using StreamHandle = void*;  // cudaStream_t
using EventHandle = void*;   // cudaEvent_t

// Seam over the few CUDA runtime calls that the host-side machinery needs, so that
// pool / token / work ordering can be tested with a fake on machines without a GPU.
class CudaResources {
 public:
  virtual ~CudaResources() = default;
  virtual int device_count() = 0;
  virtual void set_device(int index) = 0;
  virtual int current_device() = 0;
  virtual StreamHandle create_stream(int device) = 0;
  virtual void destroy_stream(int device, StreamHandle s) = 0;
  virtual EventHandle create_event(int device, bool timing) = 0;
  virtual void destroy_event(int device, EventHandle e) = 0;
  virtual void record(EventHandle e, StreamHandle s) = 0;
  virtual bool query(EventHandle e) = 0;
  virtual void wait_event_host(EventHandle e) = 0;
  virtual void stream_wait_event(StreamHandle s, EventHandle e) = 0;
  virtual void sync_stream(StreamHandle s) = 0;
  virtual float elapsed_ms(EventHandle a, EventHandle b) = 0;
  virtual void* raw_alloc(int device, size_t bytes) = 0;  // returns nullptr on OOM
  virtual void raw_free(int device, void* p) = 0;
  virtual void device_facts(int device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem) = 0;
};

std::shared_ptr<CudaResources> system_cuda_resources();

// RAII current-device switch with restore (reference: src/device/device_guard.cpp:12-58).
class DeviceGuard {
 public:
  explicit DeviceGuard(int index);
  ~DeviceGuard();
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;

 private:
  int previous_ = -1;
  bool switched_ = false;
};

// An event recorded exactly once.  An empty token counts as complete.
class CompletionToken {
 public:
  CompletionToken() = default;
  static CompletionToken record_on(int device, StreamHandle stream, bool timing = false);
  bool empty() const { return !state_; }
  bool ready() const;
  void wait_host() const;
  void enqueue_wait_on(StreamHandle stream) const;  // no-op when it is the recording stream
  float elapsed_ms_since(const CompletionToken& earlier) const;
  StreamHandle stream() const;

 private:
  struct State;
  std::shared_ptr<State> state_;
};

struct MemoryPoolStats {
  uint64_t total_requests = 0, raw_allocations = 0, reused_blocks = 0;
  uint64_t current_bytes = 0, peak_bytes = 0, cached_bytes = 0, reserved_bytes = 0;
};

class MemoryPool;

// Move-only checked-out memory.  Releases to its pool (or runs its deleter).
class Allocation {
 public:
  Allocation() = default;
  Allocation(Allocation&& o) noexcept { *this = std::move(o); }
  Allocation& operator=(Allocation&& o) noexcept;
  Allocation(const Allocation&) = delete;
  Allocation& operator=(const Allocation&) = delete;
  ~Allocation() { reset(); }

  // Wraps foreign memory (peer mappings, static device arrays, numpy-owned bytes).
  static Allocation external(void* ptr, size_t bytes, Device dev, std::function<void()> deleter);

  void* data() const { return ptr_; }
  size_t bytes() const { return bytes_; }
  size_t capacity() const { return capacity_; }
  Device device() const { return device_; }
  // Marks use by a stream other than the one the block was acquired on.
  void record_stream(StreamHandle s);
  void reset();

 private:
  friend class MemoryPool;
  void* ptr_ = nullptr;
  size_t bytes_ = 0, capacity_ = 0;
  Device device_;
  StreamHandle stream_ = nullptr;
  std::vector<StreamHandle> extra_streams_;
  MemoryPool* pool_ = nullptr;
  std::function<void()> deleter_;
};

class MemoryPool {
 public:
  static MemoryPool& instance();
  Allocation acquire(Device dev, size_t bytes, StreamHandle stream);
  void release(Allocation& a);
  // Frees every cached block (host-waits their pending events first).
  void clear();
  MemoryPoolStats stats() const;
  void reset_peak();
  void set_enabled(bool on);
  bool enabled() const { return enabled_; }
  void set_max_cached_bytes(uint64_t n);
  uint64_t max_cached_bytes() const;
  static size_t round_size(size_t bytes);

 private:
  struct Cached {
    void* ptr;
    size_t capacity;
    StreamHandle stream;
    std::vector<CompletionToken> pending;
  };
  using Key = std::pair<int, int>;  // (device type, index)
  void* raw_alloc(Device dev, size_t cap);
  void raw_free(Device dev, void* p);
  void evict_locked(uint64_t target_cached);

  mutable std::mutex mu_;
  std::map<Key, std::multimap<size_t, Cached>> free_;
  MemoryPoolStats stats_;
  bool enabled_ = true;
  uint64_t max_cached_ = ~0ull;
};

struct ScratchPoolStats {
  uint64_t leases = 0, bytes_in_use = 0, peak_bytes = 0;
};

// Exclusive kernel workspace.  A lease is pool memory on the compute stream, at least
// 1 MiB and rounded to a power of two so repeated leases hit the cache.
class ScratchLease {
 public:
  ScratchLease() = default;
  ScratchLease(Device dev, size_t bytes, StreamHandle stream);
  ~ScratchLease();
  ScratchLease(ScratchLease&&) = default;
  ScratchLease& operator=(ScratchLease&&) = default;
  void* data() const { return alloc_.data(); }
  size_t bytes() const { return alloc_.capacity(); }
  static ScratchPoolStats stats();

 private:
  Allocation alloc_;
};

class CudaContext {
 public:
  CudaContext(int device, std::shared_ptr<CudaResources> res);
  ~CudaContext();
  int device() const { return device_; }
  StreamHandle compute_stream() const { return compute_; }
  StreamHandle comm_stream() const { return comm_; }
  StreamHandle copy_stream() const { return copy_; }
  // The stream new work is issued on: the compute stream unless a StreamScope is active.
  StreamHandle current_stream() const;
  int sm_count() const { return sm_count_; }
  int cc_major() const { return cc_major_; }
  int cc_minor() const { return cc_minor_; }
  size_t total_memory() const { return total_mem_; }
  bool supports_bf16() const { return cc_major_ >= 8; }
  bool supports_tcgen05() const { return cc_major_ == 10; }
  CudaResources& resources() { return *res_; }
  std::shared_ptr<CudaResources> resources_shared() const { return res_; }
  void synchronize();

 private:
  int device_;
  std::shared_ptr<CudaResources> res_;
  StreamHandle compute_ = nullptr, comm_ = nullptr, copy_ = nullptr;
  int sm_count_ = 0, cc_major_ = 0, cc_minor_ = 0;
  size_t total_mem_ = 0;
};

class Runtime {
 public:
  static Runtime& instance();
  explicit Runtime(std::shared_ptr<CudaResources> res);
  bool cuda_available();
  int cuda_device_count();
  CudaContext& cuda(int index);
  StreamHandle stream_for(Device dev);  // nullptr for CPU
  void synchronize_all();
  CudaResources& resources() { return *res_; }
  // Replaces the CUDA seam (tests only; drops existing contexts).
  void inject_resources(std::shared_ptr<CudaResources> res);

 private:
  std::mutex mu_;
  std::shared_ptr<CudaResources> res_;
  std::vector<std::unique_ptr<CudaContext>> contexts_;
  int count_ = -1;
};

// Temporarily routes a device's new work to another stream (used for the reducer's
// communication stream and for overlapped host transfers).
class StreamScope {
 public:
  StreamScope(int device, StreamHandle s);
  ~StreamScope();
  static StreamHandle active(int device);

 private:
  int device_;
  StreamHandle prev_;
};

void cuda_check(int err, const char* what);
#define OB_CUDA(expr) ::ob::cuda_check(static_cast<int>(expr), #expr)

}  // namespace ob

// Runtime, CudaContext, CompletionToken, MemoryPool, ScratchLease.
#include "ob/runtime.h"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdlib>

namespace ob {

void cuda_check(int err, const char* what) {
  if (err != 0) {
    const cudaError_t e = static_cast<cudaError_t>(err);
    throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e) + " (" +
                             cudaGetErrorName(e) + ") in " + what);
  }
}

namespace {

class SystemCudaResources final : public CudaResources {
 public:
  int device_count() override {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    return n;
  }
  void set_device(int index) override { OB_CUDA(cudaSetDevice(index)); }
  int current_device() override {
    int d = 0;
    OB_CUDA(cudaGetDevice(&d));
    return d;
  }
  StreamHandle create_stream(int device) override {
    DeviceGuard g(device);
    cudaStream_t s;
    OB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    return s;
  }
  void destroy_stream(int device, StreamHandle s) override {
    if (s) cudaStreamDestroy(static_cast<cudaStream_t>(s));
  }
  EventHandle create_event(int device, bool timing) override {
    DeviceGuard g(device);
    cudaEvent_t e;
    OB_CUDA(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
    return e;
  }
  void destroy_event(int, EventHandle e) override {
    if (e) cudaEventDestroy(static_cast<cudaEvent_t>(e));
  }
  void record(EventHandle e, StreamHandle s) override {
    OB_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(e), static_cast<cudaStream_t>(s)));
  }
  bool query(EventHandle e) override {
    const cudaError_t r = cudaEventQuery(static_cast<cudaEvent_t>(e));
    if (r == cudaSuccess) return true;
    if (r == cudaErrorNotReady) {
      cudaGetLastError();
      return false;
    }
    OB_CUDA(r);
    return false;
  }
  void wait_event_host(EventHandle e) override { OB_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(e))); }
  void stream_wait_event(StreamHandle s, EventHandle e) override {
    OB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(s), static_cast<cudaEvent_t>(e), 0));
  }
  void sync_stream(StreamHandle s) override { OB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(s))); }
  float elapsed_ms(EventHandle a, EventHandle b) override {
    float ms = 0.f;
    OB_CUDA(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(a), static_cast<cudaEvent_t>(b)));
    return ms;
  }
  void* raw_alloc(int device, size_t bytes) override {
    DeviceGuard g(device);
    void* p = nullptr;
    const cudaError_t r = cudaMalloc(&p, bytes);
    if (r == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      return nullptr;
    }
    OB_CUDA(r);
    return p;
  }
  void raw_free(int device, void* p) override {
    DeviceGuard g(device);
    cudaFree(p);
  }
  void device_facts(int device, int* sm, int* maj, int* min, size_t* mem) override {
    cudaDeviceProp prop;
    OB_CUDA(cudaGetDeviceProperties(&prop, device));
    *sm = prop.multiProcessorCount;
    *maj = prop.major;
    *min = prop.minor;
    *mem = prop.totalGlobalMem;
  }
};

thread_local std::unordered_map<int, StreamHandle> g_stream_override;

}  // namespace

std::shared_ptr<CudaResources> system_cuda_resources() {
  static std::shared_ptr<CudaResources> r = std::make_shared<SystemCudaResources>();
  return r;
}

// ------------------------------------------------------------------ DeviceGuard
DeviceGuard::DeviceGuard(int index) {
  auto& res = Runtime::instance().resources();
  previous_ = res.current_device();
  if (previous_ != index) {
    res.set_device(index);
    switched_ = true;
  }
}

DeviceGuard::~DeviceGuard() {
  if (switched_) {
    try {
      Runtime::instance().resources().set_device(previous_);
    } catch (...) {
    }
  }
}

// -------------------------------------------------------------- CompletionToken
struct CompletionToken::State {
  int device = 0;
  StreamHandle stream = nullptr;
  EventHandle event = nullptr;
  std::shared_ptr<CudaResources> res;
  ~State() {
    if (event && res) res->destroy_event(device, event);
  }
};

CompletionToken CompletionToken::record_on(int device, StreamHandle stream, bool timing) {
  CompletionToken t;
  auto st = std::make_shared<State>();
  st->device = device;
  st->stream = stream;
  st->res = Runtime::instance().cuda(device).resources_shared();
  st->event = st->res->create_event(device, timing);
  st->res->record(st->event, stream);
  t.state_ = std::move(st);
  return t;
}

bool CompletionToken::ready() const { return !state_ || state_->res->query(state_->event); }
void CompletionToken::wait_host() const {
  if (state_) state_->res->wait_event_host(state_->event);
}
void CompletionToken::enqueue_wait_on(StreamHandle stream) const {
  if (!state_ || stream == state_->stream) return;
  state_->res->stream_wait_event(stream, state_->event);
}
float CompletionToken::elapsed_ms_since(const CompletionToken& earlier) const {
  OB_CHECK(state_ && earlier.state_, "elapsed_ms_since: both tokens must be recorded");
  state_->res->wait_event_host(state_->event);
  return state_->res->elapsed_ms(earlier.state_->event, state_->event);
}
StreamHandle CompletionToken::stream() const { return state_ ? state_->stream : nullptr; }

// ------------------------------------------------------------------- Allocation
Allocation& Allocation::operator=(Allocation&& o) noexcept {
  if (this != &o) {
    reset();
    ptr_ = o.ptr_;
    bytes_ = o.bytes_;
    capacity_ = o.capacity_;
    device_ = o.device_;
    stream_ = o.stream_;
    extra_streams_ = std::move(o.extra_streams_);
    pool_ = o.pool_;
    deleter_ = std::move(o.deleter_);
    o.ptr_ = nullptr;
    o.pool_ = nullptr;
    o.bytes_ = o.capacity_ = 0;
    o.deleter_ = nullptr;
  }
  return *this;
}

Allocation Allocation::external(void* ptr, size_t bytes, Device dev, std::function<void()> deleter) {
  Allocation a;
  a.ptr_ = ptr;
  a.bytes_ = a.capacity_ = bytes;
  a.device_ = dev;
  a.deleter_ = std::move(deleter);
  return a;
}

void Allocation::record_stream(StreamHandle s) {
  if (s == stream_) return;
  if (std::find(extra_streams_.begin(), extra_streams_.end(), s) == extra_streams_.end())
    extra_streams_.push_back(s);
}

void Allocation::reset() {
  if (pool_ && ptr_) {
    pool_->release(*this);
  } else if (deleter_) {
    auto d = std::move(deleter_);
    deleter_ = nullptr;
    try { d(); } catch (...) {}
  }
  ptr_ = nullptr;
  pool_ = nullptr;
  bytes_ = capacity_ = 0;
  extra_streams_.clear();
}

// ------------------------------------------------------------------- MemoryPool
MemoryPool& MemoryPool::instance() {
  static MemoryPool* pool = new MemoryPool();  // leaked on purpose: outlives static tensors
  return *pool;
}

size_t MemoryPool::round_size(size_t bytes) {
  if (bytes == 0) return 0;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
  return (bytes + (2u << 20) - 1) & ~size_t((2u << 20) - 1);
}

void* MemoryPool::raw_alloc(Device dev, size_t cap) {
  if (dev.is_cpu()) {
    void* p = std::aligned_alloc(64, (cap + 63) & ~size_t(63));
    if (!p) throw std::bad_alloc();
    return p;
  }
  return Runtime::instance().cuda(dev.index).resources().raw_alloc(dev.index, cap);
}

void MemoryPool::raw_free(Device dev, void* p) {
  if (dev.is_cpu()) std::free(p);
  else Runtime::instance().cuda(dev.index).resources().raw_free(dev.index, p);
}

Allocation MemoryPool::acquire(Device dev, size_t bytes, StreamHandle stream) {
  Allocation a;
  a.device_ = dev;
  a.bytes_ = bytes;
  a.stream_ = stream;
  std::unique_lock<std::mutex> lock(mu_);
  ++stats_.total_requests;
  if (bytes == 0) return a;
  const size_t cap = round_size(bytes);
  const Key key{static_cast<int>(dev.type), dev.index};
  void* ptr = nullptr;
  size_t got = cap;
  if (enabled_) {
    auto& bin = free_[key];
    // Exact size class first; otherwise the smallest block that wastes at most 1/4.
    for (auto it = bin.lower_bound(cap); it != bin.end() && it->first <= cap + cap / 4; ++it) {
      Cached& c = it->second;
      bool usable = true;
      for (auto& tok : c.pending) {
        if (tok.stream() == stream || tok.ready()) continue;
        usable = false;
        break;
      }
      if (!usable) continue;
      // The block's last owner may still have work queued on its stream that touches the block
      // (release does not record an event for the owning stream: same-stream reuse, the common
      // case, needs none).  Handing it to another stream therefore orders that stream after
      // everything the old one has queued so far: an event recorded now covers it.
      if (dev.is_cuda() && c.stream != nullptr && stream != nullptr && c.stream != stream) {
        CompletionToken::record_on(dev.index, c.stream).enqueue_wait_on(stream);
      }
      ptr = c.ptr;
      got = c.capacity;
      stats_.cached_bytes -= got;
      ++stats_.reused_blocks;
      bin.erase(it);
      break;
    }
  }
  if (!ptr) {
    lock.unlock();
    ptr = raw_alloc(dev, cap);
    if (!ptr) {  // out of device memory: drop the cache and retry once
      clear();
      ptr = raw_alloc(dev, cap);
      if (!ptr) throw std::runtime_error("out of memory allocating " + std::to_string(cap) + " bytes on " + dev.str());
    }
    lock.lock();
    ++stats_.raw_allocations;
    stats_.reserved_bytes += cap;
    got = cap;
  }
  stats_.current_bytes += got;
  stats_.peak_bytes = std::max(stats_.peak_bytes, stats_.current_bytes);
  a.ptr_ = ptr;
  a.capacity_ = got;
  a.pool_ = this;
  return a;
}

void MemoryPool::release(Allocation& a) {
  if (!a.ptr_) return;
  Cached c{a.ptr_, a.capacity_, a.stream_, {}};
  if (a.device_.is_cuda()) {
    for (StreamHandle s : a.extra_streams_) {
      try {
        c.pending.push_back(CompletionToken::record_on(a.device_.index, s));
      } catch (...) {
      }
    }
  }
  std::unique_lock<std::mutex> lock(mu_);
  stats_.current_bytes -= a.capacity_;
  if (!enabled_) {
    lock.unlock();
    if (a.device_.is_cuda()) {
      try { Runtime::instance().cuda(a.device_.index).synchronize(); } catch (...) {}
    }
    raw_free(a.device_, c.ptr);
    lock.lock();
    stats_.reserved_bytes -= c.capacity;
  } else {
    const Key key{static_cast<int>(a.device_.type), a.device_.index};
    stats_.cached_bytes += c.capacity;
    free_[key].emplace(c.capacity, std::move(c));
    if (stats_.cached_bytes > max_cached_) evict_locked(max_cached_);
  }
  a.ptr_ = nullptr;
  a.pool_ = nullptr;
}

void MemoryPool::evict_locked(uint64_t target) {
  for (auto& kv : free_) {
    auto& bin = kv.second;
    while (!bin.empty() && stats_.cached_bytes > target) {
      auto it = std::prev(bin.end());
      Cached c = std::move(it->second);
      bin.erase(it);
      const Device dev(static_cast<DeviceType>(kv.first.first), kv.first.second);
      if (dev.is_cuda()) {
        for (auto& t : c.pending) t.wait_host();
        try { Runtime::instance().cuda(dev.index).synchronize(); } catch (...) {}
      }
      raw_free(dev, c.ptr);
      stats_.cached_bytes -= c.capacity;
      stats_.reserved_bytes -= c.capacity;
    }
  }
}

void MemoryPool::clear() {
  std::lock_guard<std::mutex> lock(mu_);
  evict_locked(0);
}

MemoryPoolStats MemoryPool::stats() const {
  std::lock_guard<std::mutex> lock(mu_);
  return stats_;
}

void MemoryPool::reset_peak() {
  std::lock_guard<std::mutex> lock(mu_);
  stats_.peak_bytes = stats_.current_bytes;
}

void MemoryPool::set_enabled(bool on) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    enabled_ = on;
  }
  if (!on) clear();
}

void MemoryPool::set_max_cached_bytes(uint64_t n) {
  std::lock_guard<std::mutex> lock(mu_);
  max_cached_ = n;
  if (stats_.cached_bytes > max_cached_) evict_locked(max_cached_);
}

uint64_t MemoryPool::max_cached_bytes() const {
  std::lock_guard<std::mutex> lock(mu_);
  return max_cached_;
}

// ----------------------------------------------------------------- ScratchLease
namespace {
std::mutex g_scratch_mu;
ScratchPoolStats g_scratch_stats;
size_t scratch_round(size_t bytes) {
  size_t cap = 1u << 20;
  while (cap < bytes) cap <<= 1;
  return cap;
}
}  // namespace

ScratchLease::ScratchLease(Device dev, size_t bytes, StreamHandle stream)
    : alloc_(MemoryPool::instance().acquire(dev, scratch_round(bytes), stream)) {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  ++g_scratch_stats.leases;
  g_scratch_stats.bytes_in_use += alloc_.capacity();
  g_scratch_stats.peak_bytes = std::max(g_scratch_stats.peak_bytes, g_scratch_stats.bytes_in_use);
}

ScratchLease::~ScratchLease() {
  if (alloc_.data()) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    g_scratch_stats.bytes_in_use -= alloc_.capacity();
  }
}

ScratchPoolStats ScratchLease::stats() {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  return g_scratch_stats;
}

// ------------------------------------------------------------------ CudaContext
CudaContext::CudaContext(int device, std::shared_ptr<CudaResources> res) : device_(device), res_(std::move(res)) {
  res_->device_facts(device, &sm_count_, &cc_major_, &cc_minor_, &total_mem_);
  compute_ = res_->create_stream(device);
  comm_ = res_->create_stream(device);
  copy_ = res_->create_stream(device);
  debug_device_log("created context for cuda:" + std::to_string(device));
}

CudaContext::~CudaContext() {
  // Streams are deliberately not destroyed at process exit: the driver may already be
  // unloading, and pool blocks can still name them.
}

StreamHandle CudaContext::current_stream() const {
  StreamHandle s = StreamScope::active(device_);
  return s ? s : compute_;
}

void CudaContext::synchronize() {
  res_->sync_stream(compute_);
  res_->sync_stream(comm_);
  res_->sync_stream(copy_);
}

// ---------------------------------------------------------------------- Runtime
Runtime::Runtime(std::shared_ptr<CudaResources> res) : res_(std::move(res)) {}

Runtime& Runtime::instance() {
  static Runtime* rt = new Runtime(system_cuda_resources());
  return *rt;
}

int Runtime::cuda_device_count() {
  std::lock_guard<std::mutex> lock(mu_);
  if (count_ < 0) count_ = res_->device_count();
  return count_;
}

bool Runtime::cuda_available() { return cuda_device_count() > 0; }

CudaContext& Runtime::cuda(int index) {
  const int n = cuda_device_count();
  if (index < 0 || index >= n)
    throw std::runtime_error("CUDA device cuda:" + std::to_string(index) + " is not available (" +
                             std::to_string(n) + " visible device(s))");
  std::lock_guard<std::mutex> lock(mu_);
  if (contexts_.size() < static_cast<size_t>(n)) contexts_.resize(n);
  if (!contexts_[index]) {
    auto ctx = std::make_unique<CudaContext>(index, res_);  // published only after full init
    contexts_[index] = std::move(ctx);
  }
  return *contexts_[index];
}

StreamHandle Runtime::stream_for(Device dev) {
  if (dev.is_cpu()) return nullptr;
  return cuda(dev.index).current_stream();
}

void Runtime::synchronize_all() {
  std::vector<CudaContext*> live;
  {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& c : contexts_)
      if (c) live.push_back(c.get());
  }
  for (auto* c : live) c->synchronize();
}

void Runtime::inject_resources(std::shared_ptr<CudaResources> res) {
  MemoryPool::instance().clear();
  std::lock_guard<std::mutex> lock(mu_);
  contexts_.clear();
  res_ = std::move(res);
  count_ = -1;
}

StreamScope::StreamScope(int device, StreamHandle s) : device_(device) {
  auto it = g_stream_override.find(device);
  prev_ = it == g_stream_override.end() ? nullptr : it->second;
  g_stream_override[device] = s;
}
StreamScope::~StreamScope() { g_stream_override[device_] = prev_; }
StreamHandle StreamScope::active(int device) {
  auto it = g_stream_override.find(device);
  return it == g_stream_override.end() ? nullptr : it->second;
}

}  // namespace ob

// Ordering of records, waits and frees over a counting fake of the CUDA seam: what the pool,
// completion tokens, scratch leases and contexts promise about asynchrony, checked without a GPU.
// (reference project: tests/cpp/test_async_runtime.cpp:137-509)
#include "check.h"
#include "fake_cuda.h"
#include "ob/runtime.h"

using namespace ob;
using obtest::FakeCudaScope;

namespace {
const Device kGpu0(DeviceType::CUDA, 0), kGpu1(DeviceType::CUDA, 1);
}

TEST(async_contexts_are_created_lazily_and_once) {
  FakeCudaScope scope;
  CHECK_EQ(scope.fake->count("create_stream"), 0);
  CudaContext& a = Runtime::instance().cuda(0);
  CHECK_EQ(scope.fake->count("create_stream"), 3);
  CudaContext& b = Runtime::instance().cuda(0);
  CHECK(&a == &b);
  CHECK_EQ(scope.fake->count("create_stream"), 3);
  Runtime::instance().cuda(1);
  CHECK_EQ(scope.fake->count("create_stream"), 6);
}
TEST(async_unknown_device_is_rejected) {
  FakeCudaScope scope;
  CHECK_THROWS(Runtime::instance().cuda(2));
  CHECK_THROWS(Runtime::instance().cuda(-1));
  CHECK_EQ(Runtime::instance().cuda_device_count(), 2);
}
TEST(async_context_reports_device_facts) {
  FakeCudaScope scope;
  CudaContext& c = Runtime::instance().cuda(1);
  CHECK_EQ(c.device(), 1);
  CHECK_EQ(c.sm_count(), 148);
  CHECK(c.supports_tcgen05() && c.supports_bf16());
  CHECK_EQ(c.total_memory(), size_t(180) << 30);
  CHECK(c.compute_stream() != c.comm_stream() && c.comm_stream() != c.copy_stream());
}
TEST(async_stream_for_cpu_is_null) {
  FakeCudaScope scope;
  CHECK(Runtime::instance().stream_for(Device()) == nullptr);
  CHECK(Runtime::instance().stream_for(kGpu0) == Runtime::instance().cuda(0).compute_stream());
}
TEST(async_stream_scope_redirects_and_restores) {
  FakeCudaScope scope;
  CudaContext& c = Runtime::instance().cuda(0);
  CHECK(c.current_stream() == c.compute_stream());
  {
    StreamScope s(0, c.comm_stream());
    CHECK(c.current_stream() == c.comm_stream());
    {
      StreamScope inner(0, c.copy_stream());
      CHECK(c.current_stream() == c.copy_stream());
    }
    CHECK(c.current_stream() == c.comm_stream());
  }
  CHECK(c.current_stream() == c.compute_stream());
}
TEST(async_token_records_exactly_once) {
  FakeCudaScope scope;
  CudaContext& c = Runtime::instance().cuda(0);
  const int before = scope.fake->count("record");
  CompletionToken t = CompletionToken::record_on(0, c.compute_stream());
  CHECK_EQ(scope.fake->count("record"), before + 1);
  CompletionToken copy = t;  // copies share the event
  CHECK(copy.ready());
  CHECK_EQ(scope.fake->count("record"), before + 1);
  CHECK(t.stream() == c.compute_stream());
}
TEST(async_ready_never_waits_on_the_host) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  CudaContext& c = Runtime::instance().cuda(0);
  CompletionToken t = CompletionToken::record_on(0, c.compute_stream());
  CHECK(!t.ready());
  CHECK(!t.ready());
  CHECK_EQ(scope.fake->count("host_wait"), 0);
  t.wait_host();
  CHECK_EQ(scope.fake->count("host_wait"), 1);
  CHECK(t.ready());
}
TEST(async_wait_on_the_recording_stream_is_free) {
  FakeCudaScope scope;
  CudaContext& c = Runtime::instance().cuda(0);
  CompletionToken t = CompletionToken::record_on(0, c.comm_stream());
  t.enqueue_wait_on(c.comm_stream());
  CHECK_EQ(scope.fake->count("stream_wait"), 0);
  t.enqueue_wait_on(c.compute_stream());
  t.enqueue_wait_on(c.copy_stream());
  CHECK_EQ(scope.fake->count("stream_wait"), 2);
  CHECK_EQ(scope.fake->count("host_wait"), 0);
}
TEST(async_empty_token_is_inert) {
  FakeCudaScope scope;
  CompletionToken t;
  t.wait_host();
  t.enqueue_wait_on(Runtime::instance().cuda(0).compute_stream());
  CHECK(t.ready() && t.empty());
  CHECK_EQ(scope.fake->count("host_wait") + scope.fake->count("stream_wait"), 0);
}
TEST(async_elapsed_time_comes_from_the_seam) {
  FakeCudaScope scope;
  CudaContext& c = Runtime::instance().cuda(0);
  CompletionToken a = CompletionToken::record_on(0, c.compute_stream(), true), b = CompletionToken::record_on(0, c.compute_stream(), true);
  CHECK_NEAR(b.elapsed_ms_since(a), 1.5, 1e-6);
}
TEST(async_release_records_on_the_owning_stream_and_reuse_skips_the_wait) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  StreamHandle s = Runtime::instance().cuda(0).compute_stream();
  void* p;
  { Allocation a = pool.acquire(kGpu0, 4096, s); p = a.data(); }
  const int waits = scope.fake->count("stream_wait"), host = scope.fake->count("host_wait");
  Allocation b = pool.acquire(kGpu0, 4096, s);
  CHECK(b.data() == p);
  CHECK_EQ(scope.fake->count("stream_wait"), waits);
  CHECK_EQ(scope.fake->count("host_wait"), host);
  CHECK_EQ(scope.fake->count("raw_alloc"), 1);
}
TEST(async_reuse_on_another_stream_waits_on_the_device_not_the_host) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  CudaContext& c = Runtime::instance().cuda(0);
  void* p;
  { Allocation a = pool.acquire(kGpu0, 8192, c.compute_stream()); p = a.data(); }
  Allocation b = pool.acquire(kGpu0, 8192, c.comm_stream());
  CHECK(b.data() == p);
  CHECK(scope.fake->count("stream_wait") >= 1);
  CHECK_EQ(scope.fake->count("host_wait"), 0);
}
TEST(async_extra_stream_use_is_tracked_until_reuse) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  CudaContext& c = Runtime::instance().cuda(0);
  const int records = scope.fake->count("record");
  {
    Allocation a = pool.acquire(kGpu0, 2048, c.compute_stream());
    a.record_stream(c.comm_stream());
    a.record_stream(c.comm_stream());  // recorded once per stream
  }
  CHECK_EQ(scope.fake->count("record"), records + 1);  // one event for the foreign stream; the owning stream needs none
  const int raw = scope.fake->count("raw_alloc");
  Allocation b = pool.acquire(kGpu0, 2048, c.compute_stream());
  // The foreign use has not finished: the block is passed over (no host wait) and fresh memory is taken.
  CHECK_EQ(scope.fake->count("raw_alloc"), raw + 1);
  CHECK_EQ(scope.fake->count("host_wait"), 0);
}
TEST(async_blocks_never_cross_devices) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  void* p0;
  { Allocation a = pool.acquire(kGpu0, 4096, Runtime::instance().cuda(0).compute_stream()); p0 = a.data(); }
  Allocation b = pool.acquire(kGpu1, 4096, Runtime::instance().cuda(1).compute_stream());
  CHECK(b.data() != p0);
  CHECK_EQ(scope.fake->count("raw_alloc"), 2);
  CHECK(b.device() == kGpu1);
}
TEST(async_clear_waits_for_pending_events_before_freeing) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  { Allocation a = pool.acquire(kGpu0, 4096, Runtime::instance().cuda(0).compute_stream()); }
  scope.fake->log.clear();
  pool.clear();
  int wait_at = -1, free_at = -1;
  for (size_t i = 0; i < scope.fake->log.size(); ++i) {
    const bool waits = scope.fake->log[i] == "host_wait" || scope.fake->log[i] == "sync_stream";
    if (waits && wait_at < 0) wait_at = static_cast<int>(i);
    if (scope.fake->log[i] == "raw_free" && free_at < 0) free_at = static_cast<int>(i);
  }
  CHECK(wait_at >= 0 && free_at > wait_at);
  CHECK(scope.fake->live_blocks.empty());
}
TEST(async_eviction_waits_before_freeing) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  const uint64_t limit = pool.max_cached_bytes();
  pool.set_max_cached_bytes(0);
  { Allocation a = pool.acquire(kGpu0, 4096, Runtime::instance().cuda(0).compute_stream()); }
  CHECK_EQ(pool.stats().cached_bytes, 0u);
  CHECK(scope.fake->count("host_wait") + scope.fake->count("sync_stream") >= 1);
  CHECK_EQ(scope.fake->count("raw_free"), 1);
  pool.set_max_cached_bytes(limit);
}
TEST(async_disabled_pool_frees_after_the_owning_stream_is_done) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  pool.set_enabled(false);
  { Allocation a = pool.acquire(kGpu0, 1024, Runtime::instance().cuda(0).compute_stream()); }
  CHECK_EQ(scope.fake->count("raw_free"), 1);
  CHECK(scope.fake->count("host_wait") + scope.fake->count("sync_stream") >= 1);
  pool.set_enabled(true);
}
TEST(async_failed_allocation_unwinds_cleanly) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  const MemoryPoolStats before = pool.stats();
  scope.fake->fail_alloc = true;
  CHECK_THROWS_WITH(pool.acquire(kGpu0, size_t(1) << 20, Runtime::instance().cuda(0).compute_stream()), "out of memory");
  const MemoryPoolStats after = pool.stats();
  CHECK_EQ(after.current_bytes, before.current_bytes);
  CHECK_EQ(after.raw_allocations, before.raw_allocations);
  scope.fake->fail_alloc = false;
  Allocation ok = pool.acquire(kGpu0, size_t(1) << 20, Runtime::instance().cuda(0).compute_stream());
  CHECK(ok.data() != nullptr);
}
TEST(async_out_of_memory_retries_after_dropping_the_cache) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  StreamHandle s = Runtime::instance().cuda(0).compute_stream();
  { Allocation cached = pool.acquire(kGpu0, 4096, s); }
  CHECK(pool.stats().cached_bytes > 0);
  scope.fake->fail_alloc = true;
  CHECK_THROWS(pool.acquire(kGpu0, size_t(8) << 20, s));
  CHECK_EQ(pool.stats().cached_bytes, 0u);  // the cache was given back before giving up
  scope.fake->fail_alloc = false;
}
TEST(async_stats_follow_acquire_and_release) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  pool.reset_peak();
  const MemoryPoolStats s0 = pool.stats();
  StreamHandle s = Runtime::instance().cuda(0).compute_stream();
  {
    Allocation a = pool.acquire(kGpu0, 1000, s), b = pool.acquire(kGpu0, 3000, s);
    const MemoryPoolStats s1 = pool.stats();
    CHECK_EQ(s1.total_requests - s0.total_requests, 2u);
    CHECK_EQ(s1.current_bytes - s0.current_bytes, 1024u + 3072u);
    CHECK(s1.reserved_bytes >= s1.current_bytes);
  }
  const MemoryPoolStats s2 = pool.stats();
  CHECK_EQ(s2.current_bytes, s0.current_bytes);
  CHECK(s2.peak_bytes >= s0.current_bytes + 4096u);
  CHECK_EQ(s2.cached_bytes - s0.cached_bytes, 4096u);
}
TEST(async_scratch_lease_returns_to_the_pool_with_its_stream) {
  FakeCudaScope scope;
  StreamHandle s = Runtime::instance().cuda(0).compute_stream();
  const ScratchPoolStats before = ScratchLease::stats();
  void* p;
  {
    ScratchLease lease(kGpu0, 100, s);
    p = lease.data();
    CHECK_EQ(lease.bytes(), size_t(1) << 20);
    CHECK_EQ(ScratchLease::stats().bytes_in_use - before.bytes_in_use, uint64_t(1) << 20);
  }
  CHECK_EQ(ScratchLease::stats().bytes_in_use, before.bytes_in_use);
  CHECK_EQ(ScratchLease::stats().leases - before.leases, 1u);
  ScratchLease again(kGpu0, 5000, s);
  CHECK(again.data() == p);  // same size class: straight from the cache, no device wait on the same stream
  CHECK_EQ(scope.fake->count("stream_wait"), 0);
}
TEST(async_scratch_sizes_round_to_powers_of_two) {
  FakeCudaScope scope;
  StreamHandle s = Runtime::instance().cuda(0).compute_stream();
  CHECK_EQ(ScratchLease(kGpu0, (size_t(1) << 20) + 1, s).bytes(), size_t(2) << 20);
  CHECK_EQ(ScratchLease(kGpu0, size_t(3) << 20, s).bytes(), size_t(4) << 20);
  CHECK_EQ(ScratchLease(kGpu0, size_t(4) << 20, s).bytes(), size_t(4) << 20);
}
TEST(async_device_guard_nests) {
  FakeCudaScope scope;
  scope.fake->current = 0;
  {
    DeviceGuard outer(1);
    CHECK_EQ(scope.fake->current, 1);
    {
      DeviceGuard same(1);
      CHECK_EQ(scope.fake->current, 1);
      DeviceGuard back(0);
      CHECK_EQ(scope.fake->current, 0);
    }
    CHECK_EQ(scope.fake->current, 1);
  }
  CHECK_EQ(scope.fake->current, 0);
}
TEST(async_synchronize_all_touches_every_created_context_only) {
  FakeCudaScope scope;
  Runtime::instance().cuda(1);
  scope.fake->log.clear();
  Runtime::instance().synchronize_all();
  CHECK(scope.fake->count("sync_stream") >= 1);
  CHECK_EQ(scope.fake->count("create_stream"), 0);  // synchronising never creates a context
}
TEST(async_injecting_a_seam_drops_old_contexts_and_their_cache) {
  std::shared_ptr<obtest::FakeCuda> first;
  {
    FakeCudaScope scope;
    first = scope.fake;
    Runtime::instance().cuda(0);
    { Allocation a = MemoryPool::instance().acquire(kGpu0, 4096, Runtime::instance().cuda(0).compute_stream()); }
    CHECK_EQ(first->live_blocks.size(), 1u);
  }
  CHECK(first->live_blocks.empty());              // cached blocks went back through the seam that made them
  FakeCudaScope second;
  CHECK_EQ(second.fake->count("create_stream"), 0);  // contexts are rebuilt lazily on the new seam
  Runtime::instance().cuda(0);
  CHECK_EQ(second.fake->count("create_stream"), 3);
}

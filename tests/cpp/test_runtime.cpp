// Memory pool, allocations, completion tokens, scratch leases and contexts, on the CPU and over
// a fake CUDA seam.  (reference project: tests/cpp/test_allocator.cpp, test_async_runtime.cpp)
#include <cstring>

#include "check.h"
#include "fake_cuda.h"
#include "ob/runtime.h"

using namespace ob;
using obtest::FakeCudaScope;

namespace {
const Device kCpu(DeviceType::CPU, 0);
const Device kGpu0(DeviceType::CUDA, 0);
}  // namespace

TEST(pool_size_classes) {
  CHECK_EQ(MemoryPool::round_size(0), 0u);
  CHECK_EQ(MemoryPool::round_size(1), 512u);
  CHECK_EQ(MemoryPool::round_size(512), 512u);
  CHECK_EQ(MemoryPool::round_size(513), 1024u);
  CHECK_EQ(MemoryPool::round_size((1u << 20) + 1), size_t(2) << 20);
  CHECK_EQ(MemoryPool::round_size(size_t(5) << 20), size_t(6) << 20);
}

TEST(pool_reuses_released_cpu_blocks_and_counts) {
  MemoryPool& pool = MemoryPool::instance();
  pool.clear();
  const MemoryPoolStats s0 = pool.stats();
  void* first = nullptr;
  {
    Allocation a = pool.acquire(kCpu, 1000, nullptr);
    first = a.data();
    CHECK(first != nullptr);
    CHECK_EQ(a.bytes(), 1000u);
    CHECK_EQ(a.capacity(), 1024u);
    CHECK((reinterpret_cast<uintptr_t>(first) & 63u) == 0);
    std::memset(first, 0xAB, 1000);
    const MemoryPoolStats s1 = pool.stats();
    CHECK_EQ(s1.current_bytes - s0.current_bytes, 1024u);
    CHECK_EQ(s1.raw_allocations - s0.raw_allocations, 1u);
  }
  const MemoryPoolStats s2 = pool.stats();
  CHECK_EQ(s2.current_bytes, s0.current_bytes);
  CHECK_EQ(s2.cached_bytes - s0.cached_bytes, 1024u);
  Allocation b = pool.acquire(kCpu, 900, nullptr);  // same size class
  CHECK(b.data() == first);
  const MemoryPoolStats s3 = pool.stats();
  CHECK_EQ(s3.reused_blocks - s0.reused_blocks, 1u);
  CHECK_EQ(s3.raw_allocations - s0.raw_allocations, 1u);
  CHECK(s3.peak_bytes >= s3.current_bytes);
}

TEST(pool_zero_byte_request_is_a_null_record) {
  MemoryPool& pool = MemoryPool::instance();
  const uint64_t raw0 = pool.stats().raw_allocations;
  Allocation a = pool.acquire(kCpu, 0, nullptr);
  CHECK(a.data() == nullptr);
  CHECK_EQ(a.capacity(), 0u);
  CHECK_EQ(pool.stats().raw_allocations, raw0);
}

TEST(pool_disabled_frees_instead_of_caching) {
  MemoryPool& pool = MemoryPool::instance();
  pool.clear();
  pool.set_enabled(false);
  { Allocation a = pool.acquire(kCpu, 4096, nullptr); }
  CHECK_EQ(pool.stats().cached_bytes, 0u);
  pool.set_enabled(true);
  CHECK(pool.enabled());
}

TEST(pool_cache_limit_evicts) {
  MemoryPool& pool = MemoryPool::instance();
  pool.clear();
  const uint64_t before = pool.max_cached_bytes();
  pool.set_max_cached_bytes(2048);
  {
    Allocation a = pool.acquire(kCpu, 2048, nullptr), b = pool.acquire(kCpu, 2048, nullptr), c = pool.acquire(kCpu, 2048, nullptr);
  }
  CHECK(pool.stats().cached_bytes <= 2048u);
  pool.set_max_cached_bytes(before);
  pool.clear();
  CHECK_EQ(pool.stats().cached_bytes, 0u);
}

TEST(allocation_is_move_only_and_releases_once) {
  MemoryPool& pool = MemoryPool::instance();
  pool.clear();
  Allocation a = pool.acquire(kCpu, 100, nullptr);
  void* p = a.data();
  Allocation b = std::move(a);
  CHECK(a.data() == nullptr);
  CHECK(b.data() == p);
  const uint64_t cur = pool.stats().current_bytes;
  a.reset();  // the moved-from record owns nothing
  CHECK_EQ(pool.stats().current_bytes, cur);
  b.reset();
  CHECK_EQ(pool.stats().current_bytes, cur - 512);
  b.reset();  // idempotent
  CHECK_EQ(pool.stats().current_bytes, cur - 512);
}

TEST(external_allocation_runs_its_deleter_once) {
  int runs = 0;
  char storage[64];
  {
    Allocation a = Allocation::external(storage, sizeof(storage), kCpu, [&] { ++runs; });
    CHECK(a.data() == storage);
    Allocation b = std::move(a);
  }
  CHECK_EQ(runs, 1);
}

TEST(empty_token_is_complete) {
  CompletionToken t;
  CHECK(t.empty());
  CHECK(t.ready());
  t.wait_host();  // nothing to wait for
}

TEST(fake_cuda_context_owns_three_streams) {
  FakeCudaScope scope;
  CHECK(Runtime::instance().cuda_available());
  CHECK_EQ(Runtime::instance().cuda_device_count(), 2);
  CudaContext& ctx = Runtime::instance().cuda(0);
  CHECK_EQ(ctx.sm_count(), 148);
  CHECK(ctx.supports_tcgen05() && ctx.supports_bf16());
  CHECK(ctx.compute_stream() != nullptr && ctx.comm_stream() != nullptr && ctx.copy_stream() != nullptr);
  CHECK(ctx.compute_stream() != ctx.comm_stream());
  CHECK(ctx.current_stream() == ctx.compute_stream());
  {
    StreamScope on_comm(0, ctx.comm_stream());
    CHECK(ctx.current_stream() == ctx.comm_stream());
  }
  CHECK(ctx.current_stream() == ctx.compute_stream());
  CHECK_THROWS(Runtime::instance().cuda(7));
}

TEST(token_same_stream_needs_no_wait_and_cross_stream_waits) {
  FakeCudaScope scope;
  CudaContext& ctx = Runtime::instance().cuda(0);
  scope.fake->events_complete_immediately = false;
  CompletionToken t = CompletionToken::record_on(0, ctx.compute_stream());
  CHECK(!t.empty());
  CHECK(!t.ready());
  const int waits0 = scope.fake->count("stream_wait");
  t.enqueue_wait_on(ctx.compute_stream());
  CHECK_EQ(scope.fake->count("stream_wait"), waits0);  // the recording stream is already ordered
  t.enqueue_wait_on(ctx.comm_stream());
  CHECK_EQ(scope.fake->count("stream_wait"), waits0 + 1);
  t.wait_host();
  CHECK(t.ready());
  CHECK_EQ(scope.fake->count("host_wait"), 1);
}

TEST(device_block_reuse_on_same_stream_is_immediate) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  CudaContext& ctx = Runtime::instance().cuda(0);
  void* p = nullptr;
  {
    Allocation a = pool.acquire(kGpu0, 4096, ctx.compute_stream());
    p = a.data();
  }
  const int host_waits = scope.fake->count("host_wait");
  Allocation b = pool.acquire(kGpu0, 4096, ctx.compute_stream());
  CHECK(b.data() == p);
  CHECK_EQ(scope.fake->count("host_wait"), host_waits);  // no host wait on the hot path
  CHECK_EQ(scope.fake->count("raw_alloc"), 1);
}

TEST(device_block_used_by_another_stream_waits_for_it) {
  FakeCudaScope scope;
  scope.fake->events_complete_immediately = false;
  MemoryPool& pool = MemoryPool::instance();
  CudaContext& ctx = Runtime::instance().cuda(0);
  void* p = nullptr;
  {
    Allocation a = pool.acquire(kGpu0, 4096, ctx.compute_stream());
    p = a.data();
    a.record_stream(ctx.comm_stream());  // e.g. a collective read it
  }
  // The pending event of the communication stream has not fired: the block is not handed out.
  Allocation b = pool.acquire(kGpu0, 4096, ctx.compute_stream());
  CHECK(b.data() != p);
  CHECK_EQ(scope.fake->count("raw_alloc"), 2);
  b.reset();
  pool.clear();  // eviction host-waits the pending events before the raw free
  CHECK(scope.fake->count("host_wait") >= 1);
  CHECK(scope.fake->live_blocks.empty());
}

TEST(device_out_of_memory_is_reported_after_dropping_the_cache) {
  FakeCudaScope scope;
  MemoryPool& pool = MemoryPool::instance();
  CudaContext& ctx = Runtime::instance().cuda(0);
  { Allocation a = pool.acquire(kGpu0, 8192, ctx.compute_stream()); }
  CHECK(pool.stats().cached_bytes >= 8192u);
  scope.fake->fail_alloc = true;
  CHECK_THROWS_WITH(pool.acquire(kGpu0, size_t(64) << 20, ctx.compute_stream()), "out of memory");
  CHECK_EQ(pool.stats().cached_bytes, 0u);  // the retry emptied the cache first
  scope.fake->fail_alloc = false;
}

TEST(scratch_lease_is_at_least_one_mebibyte_and_power_of_two) {
  FakeCudaScope scope;
  CudaContext& ctx = Runtime::instance().cuda(0);
  const uint64_t leases0 = ScratchLease::stats().leases;
  {
    ScratchLease small(kGpu0, 10, ctx.compute_stream());
    CHECK(small.bytes() >= (size_t(1) << 20));
    ScratchLease odd(kGpu0, (size_t(3) << 20) + 5, ctx.compute_stream());
    CHECK_EQ(odd.bytes(), size_t(4) << 20);
    CHECK(ScratchLease::stats().bytes_in_use >= (size_t(5) << 20));
  }
  CHECK_EQ(ScratchLease::stats().leases - leases0, 2u);
  CHECK_EQ(ScratchLease::stats().bytes_in_use, 0u);
}

TEST(device_guard_restores_the_previous_device) {
  FakeCudaScope scope;
  scope.fake->current = 0;
  {
    DeviceGuard g(1);
    CHECK_EQ(scope.fake->current, 1);
    {
      DeviceGuard same(1);
      CHECK_EQ(scope.fake->current, 1);
    }
    CHECK_EQ(scope.fake->current, 1);
  }
  CHECK_EQ(scope.fake->current, 0);
}

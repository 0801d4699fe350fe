// Host-only stand-in for the CUDA seam: streams and events are small heap objects, "device"
// memory is host memory, and every call is appended to a log so that tests can assert on the
// order of records, waits and frees.  (reference project: tests/cpp/cuda_test_resources.h:4-44)
#pragma once
#include <cstdlib>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "ob/runtime.h"

namespace obtest {

class FakeCuda final : public ob::CudaResources {
 public:
  struct Event {
    bool recorded = false, complete = false;
    ob::StreamHandle stream = nullptr;
  };
  std::vector<std::string> log;
  int devices = 2;
  int current = 0;
  bool fail_alloc = false;
  bool events_complete_immediately = true;
  std::set<void*> live_blocks;

  int device_count() override { return devices; }
  void set_device(int index) override { current = index; }
  int current_device() override { return current; }
  ob::StreamHandle create_stream(int) override { log.push_back("create_stream"); return new int(0); }
  void destroy_stream(int, ob::StreamHandle s) override { log.push_back("destroy_stream"); delete static_cast<int*>(s); }
  ob::EventHandle create_event(int, bool) override { return new Event(); }
  void destroy_event(int, ob::EventHandle e) override { delete static_cast<Event*>(e); }
  void record(ob::EventHandle e, ob::StreamHandle s) override {
    auto* ev = static_cast<Event*>(e);
    ev->recorded = true;
    ev->complete = events_complete_immediately;
    ev->stream = s;
    log.push_back("record");
  }
  bool query(ob::EventHandle e) override { return static_cast<Event*>(e)->complete; }
  void wait_event_host(ob::EventHandle e) override {
    static_cast<Event*>(e)->complete = true;
    log.push_back("host_wait");
  }
  void stream_wait_event(ob::StreamHandle, ob::EventHandle) override { log.push_back("stream_wait"); }
  void sync_stream(ob::StreamHandle) override { log.push_back("sync_stream"); }
  float elapsed_ms(ob::EventHandle, ob::EventHandle) override { return 1.5f; }
  void* raw_alloc(int, size_t bytes) override {
    if (fail_alloc) return nullptr;
    void* p = std::malloc(bytes ? bytes : 1);
    live_blocks.insert(p);
    log.push_back("raw_alloc");
    return p;
  }
  void raw_free(int, void* p) override {
    live_blocks.erase(p);
    std::free(p);
    log.push_back("raw_free");
  }
  void device_facts(int, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem) override {
    *sm_count = 148; *cc_major = 10; *cc_minor = 0; *total_mem = size_t(180) << 30;
  }
  int count(const std::string& what) const {
    int n = 0;
    for (const auto& l : log) n += l == what;
    return n;
  }
};

// Installs a fake for the lifetime of the scope and restores the system seam afterwards.
struct FakeCudaScope {
  std::shared_ptr<FakeCuda> fake = std::make_shared<FakeCuda>();
  FakeCudaScope() {
    ob::MemoryPool::instance().clear();
    ob::Runtime::instance().inject_resources(fake);
  }
  ~FakeCudaScope() {
    ob::MemoryPool::instance().clear();
    ob::Runtime::instance().inject_resources(ob::system_cuda_resources());
  }
};

}  // namespace obtest

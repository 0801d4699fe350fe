// Native distributed layer: ProcessGroup / NcclProcessGroup / Work and the NCCL transport.
//
// NCCL is loaded at run time (dlopen) so the extension imports on machines without it.  One
// communicator and one communication stream per group; every collective is ordered
//   compute.record -> comm.wait -> enqueue -> bump buffer version -> comm.record -> compute.wait
// and returns a Work that owns the completion event and keeps the tensor alive.  Failures are
// sticky: the first NCCL error aborts the communicator exactly once and poisons the group.
// The transport is an injectable seam so ordering and failure handling are testable on a
// machine without GPUs (a recording fake is built in).
//
// Parity (reference project paths): src/distributed/{process_group,nccl_process_group,work,
// system_nccl_transport}.cpp, bindings/nccl_bindings.cpp:11-57.
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nccl.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <atomic>
#include <mutex>

#include "ob/ops.h"

namespace py = pybind11;

namespace ob {
namespace dist {

// ------------------------------------------------------------------ transport
class Communicator {
 public:
  virtual ~Communicator() = default;
  virtual void all_reduce(void* data, size_t count, DType dtype, StreamHandle stream) = 0;
  virtual void broadcast(void* data, size_t count, DType dtype, int src, StreamHandle stream) = 0;
  virtual std::string async_error() = 0;  // empty = healthy
  virtual void destroy() = 0;
  virtual void abort() = 0;
};

class Transport {
 public:
  virtual ~Transport() = default;
  virtual std::string unique_id() = 0;
  virtual std::unique_ptr<Communicator> init(int rank, int world, const std::string& id, int device) = 0;
};

namespace {

struct NcclApi {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) get_unique_id = nullptr;
  decltype(&ncclCommInitRank) comm_init_rank = nullptr;
  decltype(&ncclAllReduce) all_reduce = nullptr;
  decltype(&ncclBroadcast) broadcast = nullptr;
  decltype(&ncclCommGetAsyncError) get_async_error = nullptr;
  decltype(&ncclCommDestroy) comm_destroy = nullptr;
  decltype(&ncclCommAbort) comm_abort = nullptr;
  decltype(&ncclGetErrorString) error_string = nullptr;
  std::string path;
};

NcclApi& nccl_api(const std::string& preferred = "") {
  static NcclApi api;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (api.handle) return api;
  std::vector<std::string> candidates;
  if (!preferred.empty()) candidates.push_back(preferred);
  if (const char* env = std::getenv("ORTHON_NCCL_LIBRARY")) candidates.emplace_back(env);
  candidates.emplace_back("libnccl.so.2");
  candidates.emplace_back("libnccl.so");
  for (const std::string& c : candidates) {
    api.handle = dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (api.handle) { api.path = c; break; }
  }
  if (!api.handle) throw std::runtime_error("NCCL library could not be loaded (set ORTHON_NCCL_LIBRARY)");
  auto sym = [&](const char* name) {
    void* p = dlsym(api.handle, name);
    if (!p) throw std::runtime_error(std::string("NCCL symbol missing: ") + name);
    return p;
  };
  api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(sym("ncclGetUniqueId"));
  api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(sym("ncclCommInitRank"));
  api.all_reduce = reinterpret_cast<decltype(api.all_reduce)>(sym("ncclAllReduce"));
  api.broadcast = reinterpret_cast<decltype(api.broadcast)>(sym("ncclBroadcast"));
  api.get_async_error = reinterpret_cast<decltype(api.get_async_error)>(sym("ncclCommGetAsyncError"));
  api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(sym("ncclCommDestroy"));
  api.comm_abort = reinterpret_cast<decltype(api.comm_abort)>(sym("ncclCommAbort"));
  api.error_string = reinterpret_cast<decltype(api.error_string)>(sym("ncclGetErrorString"));
  return api;
}

bool nccl_loadable() {
  try {
    nccl_api();
    return true;
  } catch (...) {
    return false;
  }
}

void nccl_check(ncclResult_t r, const char* what) {
  if (r != ncclSuccess && r != ncclInProgress)
    throw std::runtime_error(std::string("NCCL error in ") + what + ": " + nccl_api().error_string(r));
}

ncclDataType_t nccl_dtype(DType d) {
  switch (d) {
    case DType::F32: return ncclFloat32;
    case DType::F16: return ncclFloat16;
    case DType::BF16: return ncclBfloat16;
    default: break;
  }
  throw std::invalid_argument(std::string("NCCL collectives support float32/float16/bfloat16, got ") + dtype_name(d));
}

class SystemCommunicator final : public Communicator {
 public:
  explicit SystemCommunicator(ncclComm_t c) : comm_(c) {}
  void all_reduce(void* data, size_t count, DType dtype, StreamHandle stream) override {
    nccl_check(nccl_api().all_reduce(data, data, count, nccl_dtype(dtype), ncclSum, comm_, static_cast<cudaStream_t>(stream)),
               "ncclAllReduce");
  }
  void broadcast(void* data, size_t count, DType dtype, int src, StreamHandle stream) override {
    nccl_check(nccl_api().broadcast(data, data, count, nccl_dtype(dtype), src, comm_, static_cast<cudaStream_t>(stream)),
               "ncclBroadcast");
  }
  std::string async_error() override {
    ncclResult_t state = ncclSuccess;
    const ncclResult_t r = nccl_api().get_async_error(comm_, &state);
    if (r != ncclSuccess) return nccl_api().error_string(r);
    if (state != ncclSuccess && state != ncclInProgress) return nccl_api().error_string(state);
    return "";
  }
  void destroy() override {
    if (comm_) nccl_api().comm_destroy(comm_);
    comm_ = nullptr;
  }
  void abort() override {
    if (comm_) nccl_api().comm_abort(comm_);
    comm_ = nullptr;
  }

 private:
  ncclComm_t comm_;
};

class SystemTransport final : public Transport {
 public:
  std::string unique_id() override {
    ncclUniqueId id;
    nccl_check(nccl_api().get_unique_id(&id), "ncclGetUniqueId");
    return std::string(id.internal, sizeof(id.internal));
  }
  std::unique_ptr<Communicator> init(int rank, int world, const std::string& id_bytes, int device) override {
    ncclUniqueId id;
    if (id_bytes.size() != sizeof(id.internal)) throw std::invalid_argument("NCCL unique id has the wrong size");
    std::memcpy(id.internal, id_bytes.data(), sizeof(id.internal));
    DeviceGuard g(device);
    ncclComm_t comm = nullptr;
    nccl_check(nccl_api().comm_init_rank(&comm, world, id, rank), "ncclCommInitRank");
    return std::make_unique<SystemCommunicator>(comm);
  }
};

// Recording fake for host-only tests: logs every call, can be told to fail.
struct FakeLog {
  std::mutex mu;
  std::vector<std::string> events;
  std::atomic<int> fail_enqueue{0}, fail_check{0};
  void add(const std::string& e) {
    std::lock_guard<std::mutex> lock(mu);
    events.push_back(e);
  }
};
FakeLog g_fake_log;

class FakeCommunicator final : public Communicator {
 public:
  void all_reduce(void*, size_t count, DType, StreamHandle) override {
    if (g_fake_log.fail_enqueue.load()) throw std::runtime_error("fake transport: injected enqueue failure");
    g_fake_log.add("all_reduce:" + std::to_string(count));
  }
  void broadcast(void*, size_t count, DType, int src, StreamHandle) override {
    if (g_fake_log.fail_enqueue.load()) throw std::runtime_error("fake transport: injected enqueue failure");
    g_fake_log.add("broadcast:" + std::to_string(count) + ":" + std::to_string(src));
  }
  std::string async_error() override { return g_fake_log.fail_check.load() ? "fake transport: injected async error" : ""; }
  void destroy() override { g_fake_log.add("destroy"); }
  void abort() override { g_fake_log.add("abort"); }
};

class FakeTransport final : public Transport {
 public:
  std::string unique_id() override { return std::string(128, 'x'); }
  std::unique_ptr<Communicator> init(int rank, int world, const std::string&, int) override {
    g_fake_log.add("init:" + std::to_string(rank) + "/" + std::to_string(world));
    return std::make_unique<FakeCommunicator>();
  }
};

// Host-only CUDA seam: streams and events are counters, memory is malloc.
class FakeCudaResources final : public CudaResources {
 public:
  explicit FakeCudaResources(int n) : n_(n) {}
  int device_count() override { return n_; }
  void set_device(int i) override { cur_ = i; }
  int current_device() override { return cur_; }
  StreamHandle create_stream(int) override { return reinterpret_cast<StreamHandle>(static_cast<uintptr_t>(++next_ * 16)); }
  void destroy_stream(int, StreamHandle) override {}
  EventHandle create_event(int, bool) override { return reinterpret_cast<EventHandle>(static_cast<uintptr_t>(++next_ * 16)); }
  void destroy_event(int, EventHandle) override {}
  void record(EventHandle e, StreamHandle s) override { g_fake_log.add("record:" + tag(e) + "@" + tag(s)); }
  bool query(EventHandle) override { return true; }
  void wait_event_host(EventHandle e) override { g_fake_log.add("host_wait:" + tag(e)); }
  void stream_wait_event(StreamHandle s, EventHandle e) override { g_fake_log.add("stream_wait:" + tag(s) + "<-" + tag(e)); }
  void sync_stream(StreamHandle s) override { g_fake_log.add("sync:" + tag(s)); }
  float elapsed_ms(EventHandle, EventHandle) override { return 0.f; }
  void* raw_alloc(int, size_t bytes) override { return std::malloc(bytes ? bytes : 1); }
  void raw_free(int, void* p) override { std::free(p); }
  void device_facts(int, int* sm, int* maj, int* min, size_t* mem) override { *sm = 148; *maj = 10; *min = 0; *mem = size_t(180) << 30; }

 private:
  static std::string tag(void* p) { return std::to_string(reinterpret_cast<uintptr_t>(p) / 16); }
  int n_, cur_ = 0;
  uintptr_t next_ = 0;
};

}  // namespace

// --------------------------------------------------------------------- groups
struct GroupLifetime {
  std::atomic<bool> closed{false};
  std::atomic<bool> failed{false};
  std::mutex mu;
  std::string failure;
  void fail(const std::string& why) {
    std::lock_guard<std::mutex> lock(mu);
    if (!failed.exchange(true)) failure = why;
  }
  std::string reason() {
    std::lock_guard<std::mutex> lock(mu);
    return failure;
  }
};

class ProcessGroup {
 public:
  ProcessGroup(int rank, int world) : rank_(rank), world_(world), life_(std::make_shared<GroupLifetime>()) {
    if (world < 1) throw std::invalid_argument("world_size must be >= 1");
    if (rank < 0 || rank >= world) throw std::invalid_argument("rank must be in [0, world_size)");
  }
  virtual ~ProcessGroup() = default;
  int rank() const { return rank_; }
  int world_size() const { return world_; }
  void ensure_open() const {
    if (life_->closed.load()) throw std::runtime_error("distributed process group has been shut down");
    if (life_->failed.load()) throw std::runtime_error("distributed process group failed: " + life_->reason());
  }

 protected:
  int rank_, world_;
  std::shared_ptr<GroupLifetime> life_;
};

// Communicator state shared by the group and its outstanding Work: abort happens once.
struct NcclStatus {
  std::unique_ptr<Communicator> comm;
  std::shared_ptr<GroupLifetime> life;
  std::mutex mu;
  bool aborted = false;
  void fail(const std::string& why) {
    life->fail(why);
    std::lock_guard<std::mutex> lock(mu);
    if (!aborted && comm) {
      aborted = true;
      try { comm->abort(); } catch (...) {}
    }
  }
  void check() {
    std::string e;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (aborted || !comm) return;
      e = comm->async_error();
    }
    if (!e.empty()) {
      fail(e);
      throw std::runtime_error("distributed process group failed: " + e);
    }
  }
};

class Work {
 public:
  Work(CompletionToken done, Tensor keep, std::shared_ptr<NcclStatus> status)
      : done_(std::move(done)), keep_(std::move(keep)), status_(std::move(status)) {}
  // Dropping a Work never waits on the host: the event and the tensor just stay alive until
  // the last reference goes away.
  bool wait() {
    if (status_->life->failed.load()) throw std::runtime_error("distributed process group failed: " + status_->life->reason());
    done_.wait_host();
    status_->check();
    keep_ = Tensor();
    return true;
  }
  bool is_completed() {
    if (status_->life->failed.load()) throw std::runtime_error("distributed process group failed: " + status_->life->reason());
    const bool ready = done_.ready();
    if (ready) status_->check();
    return ready;
  }

 private:
  CompletionToken done_;
  Tensor keep_;
  std::shared_ptr<NcclStatus> status_;
};

class NcclProcessGroup final : public ProcessGroup {
 public:
  NcclProcessGroup(int rank, int world, int device, const std::string& id, std::shared_ptr<Transport> transport)
      : ProcessGroup(rank, world), device_(device), transport_(std::move(transport)) {
    CudaContext& ctx = Runtime::instance().cuda(device);
    compute_ = ctx.compute_stream();
    comm_stream_ = ctx.comm_stream();
    status_ = std::make_shared<NcclStatus>();
    status_->life = life_;
    status_->comm = transport_->init(rank, world, id, device);
  }
  ~NcclProcessGroup() override {
    try { shutdown(); } catch (...) {}
  }

  std::shared_ptr<Work> all_reduce(Tensor& t) { return collective(t, -1); }
  std::shared_ptr<Work> broadcast(Tensor& t, int src) {
    if (src < 0 || src >= world_) throw std::invalid_argument("broadcast src must be in [0, world_size)");
    return collective(t, src);
  }
  void barrier() {
    if (!barrier_buf_.defined()) barrier_buf_ = Tensor::zeros({1}, DType::F32, Device(DeviceType::CUDA, device_));
    auto w = all_reduce(barrier_buf_);
    w->wait();
  }
  void shutdown() {
    if (life_->closed.exchange(true)) return;
    // Drain our own streams before tearing the communicator down (unless it already failed).
    if (!life_->failed.load()) {
      try {
        Runtime::instance().cuda(device_).resources().sync_stream(comm_stream_);
      } catch (...) {
      }
    }
    std::lock_guard<std::mutex> lock(status_->mu);
    if (status_->comm && !status_->aborted) {
      try { status_->comm->destroy(); } catch (...) {}
    }
    status_->comm.reset();
  }
  int device() const { return device_; }

 private:
  void validate(const Tensor& t) const {
    if (!t.device().is_cuda()) throw std::invalid_argument("NCCL collectives require CUDA tensors");
    if (t.device().index != device_)
      throw std::invalid_argument("tensor is on " + t.device().str() + " but the group was created for cuda:" + std::to_string(device_));
    if (!t.is_contiguous()) throw std::invalid_argument("NCCL collectives require contiguous tensors");
    nccl_dtype(t.dtype());
  }

  std::shared_ptr<Work> collective(Tensor& t, int src) {
    ensure_open();
    validate(t);  // preflight never mutates or poisons
    CudaResources& res = Runtime::instance().cuda(device_).resources();
    DeviceGuard guard(device_);
    // compute -> comm ordering
    CompletionToken ready = CompletionToken::record_on(device_, compute_);
    ready.enqueue_wait_on(comm_stream_);
    try {
      std::lock_guard<std::mutex> lock(status_->mu);
      if (!status_->comm || status_->aborted) throw std::runtime_error("communicator is gone");
      if (t.numel() > 0) {
        if (src < 0) status_->comm->all_reduce(t.data(), static_cast<size_t>(t.numel()), t.dtype(), comm_stream_);
        else status_->comm->broadcast(t.data(), static_cast<size_t>(t.numel()), t.dtype(), src, comm_stream_);
      }
    } catch (const std::exception& e) {
      status_->fail(e.what());
      throw std::runtime_error(std::string("distributed process group failed: ") + e.what());
    }
    t.bump_version();  // asynchronous writers count as a write at enqueue time
    t.impl()->buffer()->allocation().record_stream(comm_stream_);
    CompletionToken done = CompletionToken::record_on(device_, comm_stream_);
    done.enqueue_wait_on(compute_);  // later compute work sees the result
    (void)res;
    return std::make_shared<Work>(done, t, status_);
  }

  int device_;
  std::shared_ptr<Transport> transport_;
  std::shared_ptr<NcclStatus> status_;
  StreamHandle compute_ = nullptr, comm_stream_ = nullptr;
  Tensor barrier_buf_;
};

}  // namespace dist

void bind_peer(py::module_& m);
void bind_vmm(py::module_& m);

void bind_process_group(py::module_& m) {
  using namespace dist;
  m.def("nccl_enabled", [] { return nccl_loadable(); });
  m.def("_nccl_load", [](const std::string& path) { return nccl_api(path).path; }, py::arg("path") = "");
  m.def("_nccl_unique_id", [] { return py::bytes(SystemTransport().unique_id()); });

  py::class_<Work, std::shared_ptr<Work>>(m, "_NcclWork")
      .def("wait", &Work::wait, py::call_guard<py::gil_scoped_release>())
      .def("is_completed", &Work::is_completed);

  py::class_<NcclProcessGroup, std::shared_ptr<NcclProcessGroup>>(m, "_NcclGroup")
      .def(py::init([](int rank, int world, int device, const py::bytes& id, bool fake) {
        std::shared_ptr<Transport> tr;
        if (fake) tr = std::make_shared<FakeTransport>();
        else tr = std::make_shared<SystemTransport>();
        return std::make_shared<NcclProcessGroup>(rank, world, device, std::string(id), tr);
      }), py::arg("rank"), py::arg("world_size"), py::arg("device"), py::arg("unique_id"), py::arg("fake") = false)
      .def_property_readonly("rank", &NcclProcessGroup::rank)
      .def_property_readonly("world_size", &NcclProcessGroup::world_size)
      .def_property_readonly("device", &NcclProcessGroup::device)
      .def("ensure_open", &NcclProcessGroup::ensure_open)
      .def("all_reduce", &NcclProcessGroup::all_reduce)
      .def("broadcast", &NcclProcessGroup::broadcast)
      .def("barrier", &NcclProcessGroup::barrier, py::call_guard<py::gil_scoped_release>())
      .def("shutdown", &NcclProcessGroup::shutdown);

  // Host-only test seams.
  // Function-style access to the same group object (the spelling Orthon's private NCCL bindings use).
  using GroupPtr = std::shared_ptr<NcclProcessGroup>;
  m.def("_nccl_init", [](const py::bytes& id, int rank, int world, int device) {
    return std::make_shared<NcclProcessGroup>(rank, world, device, std::string(id), std::make_shared<SystemTransport>());
  }, py::arg("unique_id_bytes"), py::arg("rank"), py::arg("world_size"), py::arg("device_index"));
  m.def("_nccl_all_reduce_sum_async", [](const GroupPtr& group, Tensor& t) { return group->all_reduce(t); });
  m.def("_nccl_all_reduce_sum", [](const GroupPtr& group, Tensor& t) {
    auto work = group->all_reduce(t);
    py::gil_scoped_release nogil;
    work->wait();
  });
  m.def("_nccl_broadcast_async", [](const GroupPtr& group, Tensor& t, int src) { return group->broadcast(t, src); });
  m.def("_nccl_broadcast", [](const GroupPtr& group, Tensor& t, int src) {
    auto work = group->broadcast(t, src);
    py::gil_scoped_release nogil;
    work->wait();
  });
  m.def("_nccl_barrier", [](const GroupPtr& group) { group->barrier(); }, py::call_guard<py::gil_scoped_release>());
  m.def("_nccl_shutdown", [](const GroupPtr& group) { group->shutdown(); });

  m.def("_testing_use_fake_cuda", [](int devices) {
    Runtime::instance().inject_resources(devices > 0 ? std::shared_ptr<CudaResources>(std::make_shared<FakeCudaResources>(devices))
                                                     : system_cuda_resources());
  });
  m.def("_testing_fake_log", [] {
    std::lock_guard<std::mutex> lock(g_fake_log.mu);
    return g_fake_log.events;
  });
  m.def("_testing_fake_clear", [] {
    std::lock_guard<std::mutex> lock(g_fake_log.mu);
    g_fake_log.events.clear();
    g_fake_log.fail_enqueue = 0;
    g_fake_log.fail_check = 0;
  });
  m.def("_testing_fake_fail", [](bool enqueue, bool check) {
    g_fake_log.fail_enqueue = enqueue ? 1 : 0;
    g_fake_log.fail_check = check ? 1 : 0;
  });
  bind_peer(m);
  bind_vmm(m);
}

}  // namespace ob

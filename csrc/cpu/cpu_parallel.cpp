// Worker pool behind ob::cpu::parallel_for.  The pool is created on first use, is discarded
// (not joined) in a forked child so that multiprocessing workers build their own, and never
// runs nested regions in parallel.
#include "ob/cpu_parallel.h"

#include <pthread.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <mutex>
#include <thread>
#include <vector>

namespace ob {
namespace cpu {
namespace {

thread_local bool t_inside = false;

struct Pool {
  std::vector<std::thread> threads;
  std::mutex mu;
  std::condition_variable wake, done;
  const std::function<void(int64_t, int64_t)>* fn = nullptr;
  int64_t n = 0, chunk = 0;
  int parts = 0;
  uint64_t generation = 0;
  int pending = 0;
  bool stop = false;

  explicit Pool(int workers) {
    for (int w = 0; w < workers; ++w) threads.emplace_back([this, w] { loop(w + 1); });
  }
  void loop(int part) {
    uint64_t seen = 0;
    for (;;) {
      const std::function<void(int64_t, int64_t)>* f;
      int64_t lo, hi;
      {
        std::unique_lock<std::mutex> lock(mu);
        wake.wait(lock, [&] { return stop || generation != seen; });
        if (stop) return;
        seen = generation;
        if (part >= parts) continue;
        f = fn;
        lo = std::min<int64_t>(n, part * chunk);
        hi = std::min<int64_t>(n, lo + chunk);
      }
      if (lo < hi) {
        t_inside = true;  // nested regions inside a worker run inline
        (*f)(lo, hi);
        t_inside = false;
      }
      {
        std::lock_guard<std::mutex> lock(mu);
        if (--pending == 0) done.notify_one();
      }
    }
  }
};

std::mutex g_mu;
Pool* g_pool = nullptr;

void forget_pool_in_child() {
  g_pool = nullptr;  // the worker threads do not exist in the child; leak the bookkeeping
  new (&g_mu) std::mutex();
}

int configured_workers() {
  if (const char* e = std::getenv("ORTHON_CPU_THREADS")) {
    const int v = std::atoi(e);
    if (v >= 1) return v;
  }
  const unsigned hw = std::thread::hardware_concurrency();
  return static_cast<int>(std::max(1u, std::min(16u, hw ? hw : 1u)));
}

}  // namespace

int worker_count() {
  static const int n = configured_workers();
  return n;
}

void parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)>& fn) {
  if (n <= 0) return;
  const int workers = worker_count();
  int parts = static_cast<int>(std::min<int64_t>(workers, (n + std::max<int64_t>(1, grain) - 1) / std::max<int64_t>(1, grain)));
  if (parts <= 1 || t_inside) {
    fn(0, n);
    return;
  }
  std::lock_guard<std::mutex> region(g_mu);  // one parallel region at a time
  if (!g_pool) {
    static std::once_flag once;
    std::call_once(once, [] { pthread_atfork(nullptr, nullptr, forget_pool_in_child); });
    g_pool = new Pool(workers - 1);
  }
  Pool& p = *g_pool;
  const int64_t chunk = (n + parts - 1) / parts;
  {
    std::lock_guard<std::mutex> lock(p.mu);
    p.fn = &fn;
    p.n = n;
    p.chunk = chunk;
    p.parts = parts;
    p.pending = parts - 1;
    ++p.generation;
  }
  p.wake.notify_all();
  t_inside = true;
  fn(0, std::min<int64_t>(n, chunk));
  t_inside = false;
  std::unique_lock<std::mutex> lock(p.mu);
  p.done.wait(lock, [&] { return p.pending == 0; });
}

}  // namespace cpu
}  // namespace ob

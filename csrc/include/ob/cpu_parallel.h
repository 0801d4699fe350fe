// Host-side data parallelism for the CPU backend: a small persistent worker pool and a
// deterministic parallel_for (static partition, every index handled by exactly one worker in a
// fixed order, so results do not depend on the worker count).
#pragma once

#include <cstdint>
#include <functional>

namespace ob {
namespace cpu {

// Runs fn(begin, end) over [0, n) split into contiguous ranges.  Work smaller than `grain`
// indices per worker stays on the calling thread.  Nested calls run inline.
void parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)>& fn);

// Worker count (ORTHON_CPU_THREADS overrides; default min(hardware threads, 16)).
int worker_count();

}  // namespace cpu
}  // namespace ob

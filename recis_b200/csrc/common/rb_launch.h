// Counts kernel launches issued by this library (all .cu files), so that a benchmark can report how many of
// its own kernels ran inside a timed region.
#pragma once
#include <atomic>
#include <stdint.h>
namespace rb {
extern std::atomic<int64_t> g_launches;
inline void note_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
}  // namespace rb
extern "C" int64_t rb_launch_count();

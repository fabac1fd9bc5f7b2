#include "../common/rb_launch.h"
namespace rb { std::atomic<int64_t> g_launches{0}; }
extern "C" int64_t rb_launch_count() { return rb::g_launches.load(); }

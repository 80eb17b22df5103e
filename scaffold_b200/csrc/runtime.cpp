// Process-wide bookkeeping shared by the launchers.
#include <atomic>

#include "host_api.h"

static std::atomic<long long> g_launches{0};

extern "C" long long sb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" void sb_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

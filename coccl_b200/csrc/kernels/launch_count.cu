#include "launch_count.h"
#include <atomic>
static std::atomic<long> gLaunches{0};
extern "C" void cocclkCountLaunches(long n) { gLaunches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long cocclkLaunchCount(void) { return gLaunches.load(std::memory_order_relaxed); }

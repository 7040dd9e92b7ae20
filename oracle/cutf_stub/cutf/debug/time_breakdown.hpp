// Stand-in for cutf's named-timer profiler (member of the reference's exp_stats_handle,
// src/exp_stats.hpp:27; started and stopped around every statistics / scaling launch when
// profiling is enabled).  The checker never enables profiling, so the timers do nothing.
// TEST INFRASTRUCTURE ONLY, see ../math.hpp.
#pragma once
#include <string>

namespace cutf {
namespace debug {
namespace time_breakdown {
class profiler {
public:
  void start_timer_sync(const std::string &) {}
  void stop_timer_sync(const std::string &) {}
  void clear() {}
};
} // namespace time_breakdown
} // namespace debug
} // namespace cutf

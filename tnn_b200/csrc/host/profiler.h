// Thread-safe event recorder. Events carry a type (compute / communication /
// other), start and end in nanoseconds of the system clock, a name and the
// source (rank or stage) that produced them. Profilers gathered from several
// ranks are merged by shifting each one by the difference of the profilers'
// start times and sorting, and are rendered as the text line the reference's
// timeline visualiser parses (include/profiling/profiler.hpp:13-160,
// include/distributed/coordinator.hpp:465-511, visualizers/visualize_profiler.py:8).
#pragma once
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "wire.h"

namespace tnnb {

class Profiler {
 public:
  Profiler();
  void start();  // (re)set the start time to now
  int64_t start_time() const { return data_.start_time; }
  void set_start_time(int64_t t) { data_.start_time = t; }
  void add_event(uint8_t type, int64_t start_ns, int64_t end_ns, const std::string& name, const std::string& source);
  void clear();
  size_t size() const;
  std::vector<ProfEvent> events() const;
  // Shift other's events onto this profiler's time base and insert them.
  void merge(const Profiler& other);
  void sort();
  std::vector<std::string> log_lines() const;
  ProfilerData data() const;
  static std::unique_ptr<Profiler> from_data(const ProfilerData& d);
  static int64_t now_ns();

 private:
  mutable std::mutex mu_;
  ProfilerData data_;
};

}  // namespace tnnb

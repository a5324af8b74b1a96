#include "profiler.h"

#include <algorithm>
#include <chrono>
#include <cstdio>

namespace tnnb {

int64_t Profiler::now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

Profiler::Profiler() { data_.start_time = now_ns(); }

void Profiler::start() {
  std::lock_guard<std::mutex> l(mu_);
  data_.start_time = now_ns();
}

void Profiler::add_event(uint8_t type, int64_t s, int64_t e, const std::string& name, const std::string& source) {
  std::lock_guard<std::mutex> l(mu_);
  data_.events.push_back({s, e, type, name, source});
}

void Profiler::clear() {
  std::lock_guard<std::mutex> l(mu_);
  data_.events.clear();
}

size_t Profiler::size() const {
  std::lock_guard<std::mutex> l(mu_);
  return data_.events.size();
}

std::vector<ProfEvent> Profiler::events() const {
  std::lock_guard<std::mutex> l(mu_);
  return data_.events;
}

void Profiler::merge(const Profiler& other) {
  const ProfilerData od = other.data();
  std::lock_guard<std::mutex> l(mu_);
  const int64_t shift = data_.start_time - od.start_time;
  for (ProfEvent e : od.events) {
    e.start += shift;
    e.end += shift;
    data_.events.push_back(std::move(e));
  }
}

void Profiler::sort() {
  std::lock_guard<std::mutex> l(mu_);
  std::stable_sort(data_.events.begin(), data_.events.end(), [](const ProfEvent& a, const ProfEvent& b) { return a.start < b.start; });
}

std::vector<std::string> Profiler::log_lines() const {
  static const char* kTypes[] = {"COMPUTE", "COMMUNICATION", "OTHER"};
  std::lock_guard<std::mutex> l(mu_);
  std::vector<std::string> out;
  char buf[512];
  for (const auto& e : data_.events) {
    const double s = (e.start - data_.start_time) / 1e6, t = (e.end - data_.start_time) / 1e6;
    std::snprintf(buf, sizeof(buf), "Event: %s, Source: %s, Type: %s, Start: %.3f ms, End: %.3f ms, Duration: %.3f ms",
                  e.name.c_str(), e.source.c_str(), kTypes[e.type < 3 ? e.type : 2], s, t, t - s);
    out.emplace_back(buf);
  }
  return out;
}

ProfilerData Profiler::data() const {
  std::lock_guard<std::mutex> l(mu_);
  return data_;
}

std::unique_ptr<Profiler> Profiler::from_data(const ProfilerData& d) {
  auto p = std::make_unique<Profiler>();
  p->data_ = d;
  return p;
}

}  // namespace tnnb

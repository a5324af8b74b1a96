// A minimal stand-in for the part of oneTBB that the reference uses, so that its sources compile with
// USE_TBB on a machine without TBB (its code only builds in the TBB configuration: the class
// ThreadWrapper refers to its task arena unconditionally, and the OpenMP branch of thread_handler.hpp
// uses a schedule kind that g++ rejects). Written from the public oneTBB interface; nothing here is
// part of the reference. parallel_for splits the range into one contiguous piece per worker thread.
#pragma once
#include <algorithm>
#include <cstddef>
#include <thread>
#include <utility>
#include <vector>

#define TBBMALLOC_CLEAN_ALL_BUFFERS 1
inline int scalable_allocation_command(int, void*) { return 0; }

namespace tbb {

namespace detail {
inline int& arena_width() {
  static thread_local int w = 0;  // 0: outside any arena
  return w;
}
inline int workers() {
  const int w = arena_width();
  if (w > 0) return w;
  const unsigned h = std::thread::hardware_concurrency();
  return h ? static_cast<int>(h) : 1;
}
}  // namespace detail

namespace this_task_arena {
inline int max_concurrency() { return detail::workers(); }
}  // namespace this_task_arena

namespace info {
inline int default_concurrency() {
  const unsigned h = std::thread::hardware_concurrency();
  return h ? static_cast<int>(h) : 1;
}
}  // namespace info

class task_arena {
public:
  static constexpr int automatic = -1;
  explicit task_arena(int max_concurrency = automatic) : width_(max_concurrency) {}
  void initialize() {}
  void initialize(int max_concurrency) { width_ = max_concurrency; }
  void terminate() {}
  int max_concurrency() const { return width_ > 0 ? width_ : info::default_concurrency(); }
  template <typename F>
  auto execute(F&& f) -> decltype(f()) {
    struct Restore {
      int old;
      ~Restore() { detail::arena_width() = old; }
    } restore{detail::arena_width()};
    detail::arena_width() = max_concurrency();
    return f();
  }

private:
  int width_;
};

struct static_partitioner {};
struct auto_partitioner {};
struct simple_partitioner {};
struct affinity_partitioner {};

template <typename T>
class blocked_range {
public:
  using const_iterator = T;
  blocked_range(T b, T e, std::size_t grain = 1) : b_(b), e_(e), grain_(grain) {}
  T begin() const { return b_; }
  T end() const { return e_; }
  std::size_t size() const { return static_cast<std::size_t>(e_ - b_); }
  bool empty() const { return !(b_ < e_); }
  std::size_t grainsize() const { return grain_; }

private:
  T b_, e_;
  std::size_t grain_;
};

template <typename R, typename C = R>
class blocked_range2d {
public:
  blocked_range2d(R rb, R re, C cb, C ce) : rows_(rb, re), cols_(cb, ce) {}
  blocked_range2d(R rb, R re, std::size_t, C cb, C ce, std::size_t) : rows_(rb, re), cols_(cb, ce) {}
  const blocked_range<R>& rows() const { return rows_; }
  const blocked_range<C>& cols() const { return cols_; }

private:
  blocked_range<R> rows_;
  blocked_range<C> cols_;
};

namespace detail {
template <typename Body>
void run_pieces(std::size_t n, const Body& piece) {  // piece(first, last) over [0, n)
  const std::size_t w = std::min<std::size_t>(static_cast<std::size_t>(workers()), n);
  if (w <= 1) {
    if (n) piece(0, n);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(w - 1);
  const std::size_t per = (n + w - 1) / w;
  const int width = arena_width();
  for (std::size_t i = 1; i < w; ++i) {
    const std::size_t lo = i * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=, &piece] {
      arena_width() = 1;  // nested loops inside a worker run serially
      (void)width;
      piece(lo, hi);
    });
  }
  {
    const int old = arena_width();
    arena_width() = 1;
    piece(0, std::min(n, per));
    arena_width() = old;
  }
  for (auto& t : pool) t.join();
}
}  // namespace detail

template <typename T, typename Body, typename Part = auto_partitioner>
void parallel_for(const blocked_range<T>& r, const Body& body, const Part& = Part()) {
  if (r.empty()) return;
  detail::run_pieces(r.size(), [&](std::size_t lo, std::size_t hi) {
    body(blocked_range<T>(static_cast<T>(r.begin() + lo), static_cast<T>(r.begin() + hi)));
  });
}
template <typename T, typename Body>
void parallel_for(const blocked_range<T>& r, const Body& body, affinity_partitioner&) {
  parallel_for(r, body, auto_partitioner());
}

template <typename R, typename C, typename Body, typename Part = auto_partitioner>
void parallel_for(const blocked_range2d<R, C>& r, const Body& body, const Part& = Part()) {
  if (r.rows().empty() || r.cols().empty()) return;
  detail::run_pieces(r.rows().size(), [&](std::size_t lo, std::size_t hi) {
    body(blocked_range2d<R, C>(static_cast<R>(r.rows().begin() + lo), static_cast<R>(r.rows().begin() + hi),
                               r.cols().begin(), r.cols().end()));
  });
}
template <typename R, typename C, typename Body>
void parallel_for(const blocked_range2d<R, C>& r, const Body& body, affinity_partitioner&) {
  parallel_for(r, body, auto_partitioner());
}

}  // namespace tbb

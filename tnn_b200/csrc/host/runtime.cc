// Host runtime pieces that the reference implements in C++ and that stay native
// here: address-space allocators (a size-bucketed pool and a double-ended arena
// whose consecutive allocations alternate between the two ends), binary dataset
// readers with a background prefetch thread, the decode-only GPT-2 vocabulary,
// and CPU topology / affinity helpers for pinning one rank per GPU.
//
// References: include/device/pool_allocator.hpp:24-112,
// include/device/del_allocator_v2.hpp:70-426, include/data_loading/*.hpp,
// include/data_loading/batch_prefetcher.hpp:22, include/tokenizer/tokenizer.hpp:11-53,
// include/utils/thread_affinity.hpp:46-191.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <sched.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <fstream>
#include <map>
#include <mutex>
#include <random>
#include <sstream>
#include <stdexcept>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace tnnb {

// ------------------------------------------------------------------ allocators
// Both allocators hand out byte offsets inside a range the caller owns (a
// cudaMalloc'ed slab, a symmetric-heap segment, pinned host memory ...).
class PoolAllocator {
 public:
  explicit PoolAllocator(uint64_t capacity, uint64_t align = 256) : cap_(capacity), align_(align) {}
  // Reuse the smallest free block that fits, else bump.
  int64_t allocate(uint64_t bytes) {
    bytes = round(bytes);
    auto it = free_.lower_bound(bytes);
    if (it != free_.end()) {
      const uint64_t off = it->second.back();
      const uint64_t sz = it->first;
      it->second.pop_back();
      if (it->second.empty()) free_.erase(it);
      live_[off] = sz;
      used_ += sz;
      peak_ = std::max(peak_, used_);
      return (int64_t)off;
    }
    if (top_ + bytes > cap_) return -1;
    const uint64_t off = top_;
    top_ += bytes;
    live_[off] = bytes;
    used_ += bytes;
    peak_ = std::max(peak_, used_);
    return (int64_t)off;
  }
  void release(uint64_t off) {
    auto it = live_.find(off);
    if (it == live_.end()) throw std::runtime_error("PoolAllocator: release of an unknown block");
    free_[it->second].push_back(off);
    used_ -= it->second;
    live_.erase(it);
  }
  uint64_t used() const { return used_; }
  uint64_t peak() const { return peak_; }
  uint64_t reserved() const { return top_; }

 private:
  uint64_t round(uint64_t b) const { return (std::max<uint64_t>(b, 1) + align_ - 1) / align_ * align_; }
  uint64_t cap_, align_, top_ = 0, used_ = 0, peak_ = 0;
  std::map<uint64_t, std::vector<uint64_t>> free_;
  std::map<uint64_t, uint64_t> live_;
};

// Double-ended arena: side 0 grows from the left, side 1 from the right;
// flip() switches sides so that the output of layer i and the output of layer
// i+1 never fragment each other. Freed blocks are coalesced with neighbours.
class DoubleEndedArena {
 public:
  explicit DoubleEndedArena(uint64_t capacity, uint64_t align = 256) : cap_(capacity), align_(align) { free_[0] = capacity; }
  void flip() { side_ ^= 1; }
  int side() const { return side_; }
  int64_t allocate(uint64_t bytes) {
    bytes = (std::max<uint64_t>(bytes, 1) + align_ - 1) / align_ * align_;
    if (side_ == 0) {
      for (auto it = free_.begin(); it != free_.end(); ++it)
        if (it->second >= bytes) return carve(it->first, it->second, it->first, bytes);
    } else {
      for (auto it = free_.rbegin(); it != free_.rend(); ++it)
        if (it->second >= bytes) return carve(it->first, it->second, it->first + it->second - bytes, bytes);
    }
    return -1;
  }
  void release(uint64_t off) {
    auto it = live_.find(off);
    if (it == live_.end()) throw std::runtime_error("DoubleEndedArena: release of an unknown block");
    uint64_t start = off, size = it->second;
    used_ -= size;
    live_.erase(it);
    auto nx = free_.lower_bound(start);
    if (nx != free_.end() && start + size == nx->first) {
      size += nx->second;
      nx = free_.erase(nx);
    }
    if (nx != free_.begin()) {
      auto pv = std::prev(nx);
      if (pv->first + pv->second == start) {
        start = pv->first;
        size += pv->second;
        free_.erase(pv);
      }
    }
    free_[start] = size;
  }
  void reset() {
    live_.clear();
    free_.clear();
    free_[0] = cap_;
    used_ = 0;
  }
  uint64_t used() const { return used_; }
  uint64_t peak() const { return peak_; }
  size_t free_blocks() const { return free_.size(); }

 private:
  int64_t carve(uint64_t blk_off, uint64_t blk_size, uint64_t off, uint64_t bytes) {
    free_.erase(blk_off);
    if (off > blk_off) free_[blk_off] = off - blk_off;
    if (off + bytes < blk_off + blk_size) free_[off + bytes] = blk_off + blk_size - (off + bytes);
    live_[off] = bytes;
    used_ += bytes;
    peak_ = std::max(peak_, used_);
    return (int64_t)off;
  }
  uint64_t cap_, align_, used_ = 0, peak_ = 0;
  int side_ = 0;
  std::map<uint64_t, uint64_t> free_, live_;
};

// ---------------------------------------------------------------- data loaders
struct Batch {
  py::array_t<float> data;
  py::array_t<int32_t> labels;
};

class Dataset {
 public:
  virtual ~Dataset() = default;
  virtual size_t size() const = 0;
  virtual std::vector<size_t> sample_shape() const = 0;
  // Write sample i (float, channels-last) and return its label(s).
  virtual void fetch(size_t i, float* out, int32_t* label, std::mt19937_64& rng) const = 0;
  virtual size_t labels_per_sample() const { return 1; }
};

// CIFAR-10: records of 1 label byte + 3072 bytes CHW u8. CIFAR-100: coarse, fine, 3072 bytes.
class CifarDataset : public Dataset {
 public:
  CifarDataset(const std::vector<std::string>& files, bool cifar100, bool coarse) {
    const size_t rec = cifar100 ? 3074 : 3073;
    for (const auto& f : files) {
      std::ifstream in(f, std::ios::binary);
      if (!in) throw std::runtime_error("cannot open " + f);
      std::stringstream ss;
      ss << in.rdbuf();
      const std::string b = ss.str();
      if (b.size() % rec) throw std::runtime_error(f + ": size is not a multiple of the record length");
      for (size_t o = 0; o + rec <= b.size(); o += rec) {
        labels_.push_back(cifar100 ? (uint8_t)b[o + (coarse ? 0 : 1)] : (uint8_t)b[o]);
        pixels_.insert(pixels_.end(), b.begin() + o + (cifar100 ? 2 : 1), b.begin() + o + rec);
      }
    }
  }
  size_t size() const override { return labels_.size(); }
  std::vector<size_t> sample_shape() const override { return {32, 32, 3}; }
  void fetch(size_t i, float* out, int32_t* label, std::mt19937_64&) const override {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(pixels_.data()) + i * 3072;
    for (int c = 0; c < 3; ++c)
      for (int hw = 0; hw < 1024; ++hw) out[hw * 3 + c] = p[c * 1024 + hw] / 255.f;
    *label = labels_[i];
  }

 private:
  std::vector<uint8_t> labels_;
  std::string pixels_;
};

// MNIST CSV with a header line: label,p0..p783 ; pixels / 255.
class MnistCsvDataset : public Dataset {
 public:
  explicit MnistCsvDataset(const std::string& path) {
    std::ifstream in(path);
    if (!in) throw std::runtime_error("cannot open " + path);
    std::string line;
    std::getline(in, line);  // header
    while (std::getline(in, line)) {
      if (line.empty()) continue;
      const char* s = line.c_str();
      char* e;
      labels_.push_back((int32_t)std::strtol(s, &e, 10));
      for (int k = 0; k < 784; ++k) {
        if (*e == ',') ++e;
        pixels_.push_back((uint8_t)std::strtol(e, &e, 10));
      }
    }
  }
  size_t size() const override { return labels_.size(); }
  std::vector<size_t> sample_shape() const override { return {28, 28, 1}; }
  void fetch(size_t i, float* out, int32_t* label, std::mt19937_64&) const override {
    for (int k = 0; k < 784; ++k) out[k] = pixels_[i * 784 + k] / 255.f;
    *label = labels_[i];
  }

 private:
  std::vector<int32_t> labels_;
  std::vector<uint8_t> pixels_;
};

// Flat uint16 token stream; a sample is a random window of ctx tokens, labels are the
// same window shifted by one. Token ids are emitted as floats holding exact integers.
class TokenDataset : public Dataset {
 public:
  TokenDataset(const std::string& path, size_t ctx) : ctx_(ctx) {
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in) throw std::runtime_error("cannot open " + path);
    const size_t bytes = (size_t)in.tellg();
    in.seekg(0);
    tokens_.resize(bytes / 2);
    in.read(reinterpret_cast<char*>(tokens_.data()), (std::streamsize)(tokens_.size() * 2));
    if (tokens_.size() < ctx + 1) throw std::runtime_error(path + ": fewer tokens than one context window");
  }
  size_t size() const override { return tokens_.size() / ctx_; }
  std::vector<size_t> sample_shape() const override { return {ctx_}; }
  size_t labels_per_sample() const override { return ctx_; }
  void fetch(size_t, float* out, int32_t* label, std::mt19937_64& rng) const override {
    std::uniform_int_distribution<size_t> d(0, tokens_.size() - ctx_ - 1);
    const size_t o = d(rng);
    for (size_t k = 0; k < ctx_; ++k) {
      out[k] = (float)tokens_[o + k];
      label[k] = tokens_[o + k + 1];
    }
  }

 private:
  size_t ctx_;
  std::vector<uint16_t> tokens_;
};

// Shuffling batcher with an optional background thread that keeps `depth` batches ready.
class Loader {
 public:
  Loader(std::shared_ptr<Dataset> ds, size_t batch, bool shuffle, uint64_t seed, size_t prefetch_depth)
      : ds_(std::move(ds)), batch_(batch), shuffle_(shuffle), rng_(seed), depth_(prefetch_depth) {
    order_.resize(ds_->size());
    for (size_t i = 0; i < order_.size(); ++i) order_[i] = i;
    reset();
  }
  ~Loader() { stop(); }
  size_t size() const { return ds_->size(); }
  size_t batches_per_epoch() const { return ds_->size() / batch_; }
  std::vector<size_t> sample_shape() const { return ds_->sample_shape(); }

  void reset() {
    stop();
    if (shuffle_) std::shuffle(order_.begin(), order_.end(), rng_);
    cursor_ = 0;
    if (depth_ > 0) {
      running_ = true;
      worker_ = std::thread([this] { run(); });
    }
  }

  // Returns false at the end of the epoch.
  bool next(std::vector<float>& data, std::vector<int32_t>& labels) {
    if (depth_ == 0) return produce(data, labels);
    std::unique_lock<std::mutex> l(mu_);
    cv_.wait(l, [this] { return !queue_.empty() || done_; });
    if (queue_.empty()) return false;
    data = std::move(queue_.front().first);
    labels = std::move(queue_.front().second);
    queue_.pop_front();
    cv_.notify_all();
    return true;
  }

  size_t batch() const { return batch_; }
  size_t labels_per_sample() const { return ds_->labels_per_sample(); }

 private:
  bool produce(std::vector<float>& data, std::vector<int32_t>& labels) {
    if (cursor_ + batch_ > order_.size()) return false;
    size_t per = 1;
    for (size_t d : ds_->sample_shape()) per *= d;
    const size_t lps = ds_->labels_per_sample();
    data.resize(batch_ * per);
    labels.resize(batch_ * lps);
    for (size_t b = 0; b < batch_; ++b) ds_->fetch(order_[cursor_ + b], data.data() + b * per, labels.data() + b * lps, rng_);
    cursor_ += batch_;
    return true;
  }
  void run() {
    for (;;) {
      std::vector<float> d;
      std::vector<int32_t> lab;
      const bool ok = produce(d, lab);
      std::unique_lock<std::mutex> l(mu_);
      if (!ok) {
        done_ = true;
        cv_.notify_all();
        return;
      }
      cv_.wait(l, [this] { return queue_.size() < depth_ || !running_; });
      if (!running_) return;
      queue_.emplace_back(std::move(d), std::move(lab));
      cv_.notify_all();
    }
  }
  void stop() {
    {
      std::lock_guard<std::mutex> l(mu_);
      running_ = false;
      cv_.notify_all();
    }
    if (worker_.joinable()) worker_.join();
    queue_.clear();
    done_ = false;
  }

  std::shared_ptr<Dataset> ds_;
  size_t batch_;
  bool shuffle_;
  std::mt19937_64 rng_;
  size_t depth_;
  std::vector<size_t> order_;
  size_t cursor_ = 0;
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::pair<std::vector<float>, std::vector<int32_t>>> queue_;
  bool running_ = false, done_ = false;
};

// ------------------------------------------------------------------- tokenizer
// vocab.bin = u32 n, then n x (u32 len, bytes). Decode only.
class Tokenizer {
 public:
  explicit Tokenizer(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("cannot open " + path);
    uint32_t n = 0;
    in.read(reinterpret_cast<char*>(&n), 4);
    vocab_.resize(n);
    for (uint32_t i = 0; i < n; ++i) {
      uint32_t len = 0;
      in.read(reinterpret_cast<char*>(&len), 4);
      vocab_[i].resize(len);
      in.read(vocab_[i].data(), len);
      if (!in) throw std::runtime_error(path + ": truncated vocabulary");
    }
  }
  size_t size() const { return vocab_.size(); }
  py::bytes token(size_t i) const { return py::bytes(i < vocab_.size() ? vocab_[i] : std::string()); }
  py::bytes decode(const std::vector<int64_t>& ids) const {
    std::string s;
    for (int64_t i : ids)
      if (i >= 0 && (size_t)i < vocab_.size()) s += vocab_[(size_t)i];
    return py::bytes(s);
  }

 private:
  std::vector<std::string> vocab_;
};

// -------------------------------------------------------------- cpu / affinity
static py::dict hardware_info() {
  py::dict d;
  d["logical_cpus"] = (long)sysconf(_SC_NPROCESSORS_ONLN);
  d["page_size"] = (long)sysconf(_SC_PAGESIZE);
  d["phys_pages"] = (long)sysconf(_SC_PHYS_PAGES);
  cpu_set_t set;
  CPU_ZERO(&set);
  std::vector<int> allowed;
  if (sched_getaffinity(0, sizeof(set), &set) == 0)
    for (int i = 0; i < CPU_SETSIZE; ++i)
      if (CPU_ISSET(i, &set)) allowed.push_back(i);
  d["allowed_cpus"] = allowed;
  std::ifstream f("/proc/cpuinfo");
  std::string line;
  while (std::getline(f, line))
    if (line.rfind("model name", 0) == 0) {
      d["model_name"] = line.substr(line.find(':') + 2);
      break;
    }
  return d;
}

// Pin the calling thread to the k-th slice of the allowed CPUs (one slice per local rank).
static std::vector<int> pin_rank(int local_rank, int local_world) {
  cpu_set_t set;
  CPU_ZERO(&set);
  std::vector<int> allowed;
  if (sched_getaffinity(0, sizeof(set), &set) != 0) return {};
  for (int i = 0; i < CPU_SETSIZE; ++i)
    if (CPU_ISSET(i, &set)) allowed.push_back(i);
  if (local_world <= 0 || allowed.empty()) return {};
  const size_t per = std::max<size_t>(1, allowed.size() / (size_t)local_world);
  const size_t b = std::min(allowed.size() - 1, (size_t)local_rank * per);
  const size_t e = std::min(allowed.size(), b + per);
  cpu_set_t mine;
  CPU_ZERO(&mine);
  std::vector<int> out;
  for (size_t i = b; i < e; ++i) {
    CPU_SET(allowed[i], &mine);
    out.push_back(allowed[i]);
  }
  if (sched_setaffinity(0, sizeof(mine), &mine) != 0) return {};
  return out;
}

void bind_runtime(py::module_& m) {
  py::class_<PoolAllocator>(m, "PoolAllocator")
      .def(py::init<uint64_t, uint64_t>(), py::arg("capacity"), py::arg("align") = 256)
      .def("allocate", &PoolAllocator::allocate)
      .def("release", &PoolAllocator::release)
      .def("used", &PoolAllocator::used)
      .def("peak", &PoolAllocator::peak)
      .def("reserved", &PoolAllocator::reserved);
  py::class_<DoubleEndedArena>(m, "DoubleEndedArena")
      .def(py::init<uint64_t, uint64_t>(), py::arg("capacity"), py::arg("align") = 256)
      .def("allocate", &DoubleEndedArena::allocate)
      .def("release", &DoubleEndedArena::release)
      .def("flip", &DoubleEndedArena::flip)
      .def("side", &DoubleEndedArena::side)
      .def("reset", &DoubleEndedArena::reset)
      .def("used", &DoubleEndedArena::used)
      .def("peak", &DoubleEndedArena::peak)
      .def("free_blocks", &DoubleEndedArena::free_blocks);

  py::class_<Loader>(m, "Loader")
      .def_static("cifar10", [](const std::vector<std::string>& files, size_t batch, bool shuffle, uint64_t seed, size_t depth) {
        return std::make_unique<Loader>(std::make_shared<CifarDataset>(files, false, false), batch, shuffle, seed, depth);
      })
      .def_static("cifar100", [](const std::vector<std::string>& files, bool coarse, size_t batch, bool shuffle, uint64_t seed, size_t depth) {
        return std::make_unique<Loader>(std::make_shared<CifarDataset>(files, true, coarse), batch, shuffle, seed, depth);
      })
      .def_static("mnist_csv", [](const std::string& path, size_t batch, bool shuffle, uint64_t seed, size_t depth) {
        return std::make_unique<Loader>(std::make_shared<MnistCsvDataset>(path), batch, shuffle, seed, depth);
      })
      .def_static("tokens", [](const std::string& path, size_t ctx, size_t batch, uint64_t seed, size_t depth) {
        return std::make_unique<Loader>(std::make_shared<TokenDataset>(path, ctx), batch, true, seed, depth);
      })
      .def("__len__", &Loader::size)
      .def("batches_per_epoch", &Loader::batches_per_epoch)
      .def("sample_shape", &Loader::sample_shape)
      .def("reset", &Loader::reset, py::call_guard<py::gil_scoped_release>())
      .def("next", [](Loader& l) -> py::object {
        std::vector<float> d;
        std::vector<int32_t> lab;
        bool ok;
        {
          py::gil_scoped_release rel;
          ok = l.next(d, lab);
        }
        if (!ok) return py::none();
        std::vector<py::ssize_t> shape{(py::ssize_t)l.batch()};
        for (size_t s : l.sample_shape()) shape.push_back((py::ssize_t)s);
        py::array_t<float> a(shape);
        std::memcpy(a.mutable_data(), d.data(), d.size() * 4);
        std::vector<py::ssize_t> lshape{(py::ssize_t)l.batch()};
        if (l.labels_per_sample() > 1) lshape.push_back((py::ssize_t)l.labels_per_sample());
        py::array_t<int32_t> b(lshape);
        std::memcpy(b.mutable_data(), lab.data(), lab.size() * 4);
        return py::make_tuple(a, b);
      });

  py::class_<Tokenizer>(m, "Tokenizer")
      .def(py::init<const std::string&>())
      .def("__len__", &Tokenizer::size)
      .def("token", &Tokenizer::token)
      .def("decode", &Tokenizer::decode);

  m.def("hardware_info", &hardware_info);
  m.def("pin_rank", &pin_rank, py::arg("local_rank"), py::arg("local_world"));
}

}  // namespace tnnb

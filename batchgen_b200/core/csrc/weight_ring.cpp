// WeightRing implementation + the two copy backends.  See weight_ring.h.
#include "weight_ring.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cstdlib>
#include <cstring>

namespace bgcore {

// ------------------------------------------------------------------ host backend (tests, CPU runs)
namespace {
struct HostBackend : CopyBackend {
  void* alloc_device(size_t bytes) override { return std::malloc(bytes ? bytes : 1); }
  void free_device(void* p) override { std::free(p); }
  void copy_h2d_async(void* dst, const void* src, size_t bytes) override { std::memcpy(dst, src, bytes); }
  void* record_producer_event() override { return reinterpret_cast<void*>(1); }
  void* record_stream_event(void*) override { return reinterpret_cast<void*>(1); }
  bool event_done(void*) override { return true; }
  void destroy_event(void*) override {}
  bool pin_host(void*, size_t) override { return true; }
  void unpin_host(void*) override {}
};

struct CudaBackend : CopyBackend {
  int device;
  cudaStream_t stream = nullptr;
  explicit CudaBackend(int dev) : device(dev) {}
  bool init() {
    if (cudaSetDevice(device) != cudaSuccess) return false;
    return cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess;
  }
  ~CudaBackend() override {
    if (stream) cudaStreamDestroy(stream);
  }
  void* alloc_device(size_t bytes) override {
    void* p = nullptr;
    cudaSetDevice(device);
    return cudaMalloc(&p, bytes) == cudaSuccess ? p : nullptr;
  }
  void free_device(void* p) override { cudaFree(p); }
  void copy_h2d_async(void* dst, const void* src, size_t bytes) override {
    cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);   // one copy per tensor
  }
  void* record_producer_event() override {
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, stream);
    return ev;
  }
  void* record_stream_event(void* s) override {
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, reinterpret_cast<cudaStream_t>(s));
    return ev;
  }
  bool event_done(void* ev) override { return cudaEventQuery(reinterpret_cast<cudaEvent_t>(ev)) != cudaErrorNotReady; }
  void destroy_event(void* ev) override { cudaEventDestroy(reinterpret_cast<cudaEvent_t>(ev)); }
  bool pin_host(void* p, size_t bytes) override {
    return cudaHostRegister(p, bytes, cudaHostRegisterDefault) == cudaSuccess;
  }
  void unpin_host(void* p) override { cudaHostUnregister(p); }
};
}  // namespace

std::unique_ptr<CopyBackend> make_host_backend() { return std::unique_ptr<CopyBackend>(new HostBackend()); }

std::unique_ptr<CopyBackend> make_cuda_backend(int device) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device >= n) return nullptr;
  std::unique_ptr<CudaBackend> b(new CudaBackend(device));
  if (!b->init()) return nullptr;
  return std::unique_ptr<CopyBackend>(b.release());
}

// ------------------------------------------------------------------ ring
WeightRing::WeightRing(int num_slots, size_t slot_bytes, std::unique_ptr<CopyBackend> backend)
    : be_(std::move(backend)), slot_bytes_(slot_bytes), table_(num_slots) {
  for (int i = 0; i < num_slots; ++i) slots_.push_back(be_->alloc_device(slot_bytes));
}

WeightRing::~WeightRing() {
  stop_producer();
  drain(true);
  for (void* p : slots_) be_->free_device(p);
}

bool WeightRing::register_module(int module, std::vector<TensorSpan>* spans) {
  size_t off = 0;
  for (auto& t : *spans) {
    off = (off + 255) & ~size_t(255);
    t.slot_offset = off;
    off += t.bytes;
  }
  if (off > slot_bytes_) return false;
  std::lock_guard<std::mutex> lk(mu_);
  modules_[module] = *spans;
  return true;
}

void WeightRing::install_queue(const std::vector<int>& modules) {
  std::lock_guard<std::mutex> lk(mu_);
  table_.install_queue(modules);
  aborted_ = false;
}

uint64_t WeightRing::begin_pass(bool carry) {
  std::lock_guard<std::mutex> lk(mu_);
  aborted_ = false;
  uint64_t id = table_.begin_pass(carry);
  cv_producer_.notify_all();
  return id;
}

bool WeightRing::end_pass() {
  std::lock_guard<std::mutex> lk(mu_);
  bool ok = table_.end_pass();
  cv_producer_.notify_all();
  return ok;
}

void WeightRing::skip_modules(const std::vector<int>& modules) {
  std::lock_guard<std::mutex> lk(mu_);
  table_.skip_modules(modules);
  cv_consumer_.notify_all();
}

void WeightRing::abort_passes() {
  std::lock_guard<std::mutex> lk(mu_);
  aborted_ = true;
  table_.abort_all();
  cv_consumer_.notify_all();
  cv_producer_.notify_all();
}

void WeightRing::start_producer() {
  if (running_.exchange(true)) return;
  thread_ = std::thread([this] { producer_loop(); });
}

void WeightRing::stop_producer() {
  if (!running_.exchange(false)) return;
  cv_producer_.notify_all();
  if (thread_.joinable()) thread_.join();
}

// Complete landings and reclaim released slots whose events have fired.
void WeightRing::drain(bool all) {
  std::unique_lock<std::mutex> lk(mu_);
  bool changed = false;
  while (!landings_.empty() && (all || be_->event_done(landings_.front().ev))) {
    Landing l = landings_.front();
    landings_.pop_front();
    be_->destroy_event(l.ev);
    table_.landed(l.slot);
    changed = true;
  }
  for (size_t i = 0; i < releases_.size();) {
    if (all || be_->event_done(releases_[i].ev)) {
      be_->destroy_event(releases_[i].ev);
      table_.reclaim(releases_[i].slot);
      releases_.erase(releases_.begin() + i);
      changed = true;
    } else {
      ++i;
    }
  }
  if (changed) {
    cv_consumer_.notify_all();
    cv_producer_.notify_all();
  }
}

void WeightRing::producer_loop() {
  while (running_) {
    drain(false);
    Production pr;
    std::vector<TensorSpan> spans;
    bool have = false;
    {
      std::unique_lock<std::mutex> lk(mu_);
      if (static_cast<int>(landings_.size()) < kMaxInFlight && table_.next_production(&pr)) {
        auto it = modules_.find(pr.module);
        if (it != modules_.end()) spans = it->second;
        have = true;
      } else {
        cv_producer_.wait_for(lk, std::chrono::microseconds(200));
      }
    }
    if (!have) continue;
    auto t0 = std::chrono::steady_clock::now();
    uint64_t bytes = 0;
    for (const auto& t : spans) {
      be_->copy_h2d_async(static_cast<char*>(slots_[pr.slot]) + t.slot_offset, t.host, t.bytes);
      bytes += t.bytes;
    }
    void* ev = be_->record_producer_event();
    auto t1 = std::chrono::steady_clock::now();
    {
      std::lock_guard<std::mutex> lk(mu_);
      landings_.push_back({pr.slot, ev});
      stats_.modules_copied += 1;
      stats_.bytes_copied += bytes;
      stats_.copy_seconds += std::chrono::duration<double>(t1 - t0).count();
    }
  }
}

void* WeightRing::get_weights(int module, int timeout_ms, int* slot_out) {
  auto t0 = std::chrono::steady_clock::now();
  auto deadline = t0 + std::chrono::milliseconds(timeout_ms);
  std::unique_lock<std::mutex> lk(mu_);
  stats_.get_calls += 1;
  while (true) {
    if (aborted_) return nullptr;
    int s = table_.acquire(module);
    if (s >= 0) {
      if (slot_out) *slot_out = s;
      stats_.get_wait_us +=
          std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
      return slots_[s];
    }
    if (s == -2) return nullptr;   // not the module the pass expects next
    if (std::chrono::steady_clock::now() >= deadline) {
      stats_.stalls += 1;
      return nullptr;
    }
    lk.unlock();
    if (!running_) drain(false);   // no producer thread (tests drive the ring by hand)
    lk.lock();
    cv_consumer_.wait_for(lk, std::chrono::microseconds(200));
  }
}

void WeightRing::release(int slot, void* consumer_stream) {
  std::lock_guard<std::mutex> lk(mu_);
  if (consumer_stream == nullptr) {
    table_.release(slot, false);
  } else {
    table_.release(slot, true);
    releases_.push_back({slot, be_->record_stream_event(consumer_stream)});
  }
  cv_producer_.notify_all();
}

RingStats WeightRing::stats() {
  std::lock_guard<std::mutex> lk(mu_);
  RingStats s = stats_;
  s.modules_skipped = table_.skipped_total();
  return s;
}

int WeightRing::count_state(int st) {
  std::lock_guard<std::mutex> lk(mu_);
  return table_.count(static_cast<SlotState>(st));
}

}  // namespace bgcore

// WeightRing: a ring of device weight slots fed by a producer thread from host memory.
//
// The consumer (the model's forward pass) calls get_weights(module) which blocks (bounded) until the
// producer has landed that module in a slot, computes with the returned device pointer, and releases
// the slot, synchronously or on an event of its compute stream.  The producer walks the installed
// forward-order queue pass after pass, claims FREE slots (WeightSlotTable), issues one asynchronous
// host->device copy per tensor on its own non-blocking stream, and marks the slot PRESENT when the
// copy's event completes ("event-deferred landing"; at most kMaxInFlight copies are outstanding).
//
// Copies go through a CopyBackend so that the whole ring — threads, passes, skips, aborts, stall
// bound — runs and is tested without a GPU (HostBackend = memcpy); CudaBackend uses cudaMemcpyAsync,
// cudaEvent and pinned host registrations.
//
// Reference parity: core/GPU_Weight_Buffer/GPU_Weight_Buffer.h:53-245 (slot ring, get_weights with a
// 300 s stall bound, passes, async release on consumer-stream events), core/HtoD_Engine/HtoD_Engine.h:49-393
// (producer thread on a non-blocking stream, event-deferred landings <= 64 in flight, per-type
// statistics).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "weight_slot_table.h"

namespace bgcore {

struct CopyBackend {
  virtual ~CopyBackend() {}
  virtual void* alloc_device(size_t bytes) = 0;
  virtual void free_device(void* p) = 0;
  virtual void copy_h2d_async(void* dst, const void* src, size_t bytes) = 0;   // on the producer stream
  virtual void* record_producer_event() = 0;                                   // after the copies above
  virtual void* record_stream_event(void* stream) = 0;                         // on a consumer stream
  virtual bool event_done(void* ev) = 0;
  virtual void destroy_event(void* ev) = 0;
  virtual bool pin_host(void* p, size_t bytes) = 0;
  virtual void unpin_host(void* p) = 0;
};

std::unique_ptr<CopyBackend> make_host_backend();
std::unique_ptr<CopyBackend> make_cuda_backend(int device);   // nullptr when CUDA is unusable

struct TensorSpan {
  const void* host;
  size_t bytes;
  size_t slot_offset;   // filled by register_module
};

struct RingStats {
  uint64_t modules_copied = 0, modules_skipped = 0, bytes_copied = 0;
  uint64_t get_calls = 0, get_wait_us = 0, stalls = 0;
  double copy_seconds = 0.0;
};

constexpr int kMaxInFlight = 64;

class WeightRing {
 public:
  WeightRing(int num_slots, size_t slot_bytes, std::unique_ptr<CopyBackend> backend);
  ~WeightRing();

  // Tensors of a module are packed back to back (256-byte aligned) inside a slot.  Returns the slot
  // offsets through `spans`, or false if the module does not fit a slot.
  bool register_module(int module, std::vector<TensorSpan>* spans);
  void install_queue(const std::vector<int>& modules);
  uint64_t begin_pass(bool carry);
  bool end_pass();
  void skip_modules(const std::vector<int>& modules);
  void abort_passes();

  void start_producer();
  void stop_producer();

  // Device base pointer of the slot holding `module` (nullptr on timeout / abort / out-of-order).
  void* get_weights(int module, int timeout_ms, int* slot_out);
  void release(int slot, void* consumer_stream);   // stream == nullptr: synchronous release

  RingStats stats();
  size_t slot_bytes() const { return slot_bytes_; }
  int num_slots() const { return table_.num_slots(); }
  void* slot_ptr(int slot) const { return slots_[slot]; }
  int count_state(int st);

 private:
  void producer_loop();
  void drain(bool all);

  struct Landing { int slot; void* ev; };
  struct PendingRelease { int slot; void* ev; };

  std::unique_ptr<CopyBackend> be_;
  size_t slot_bytes_;
  std::vector<void*> slots_;
  WeightSlotTable table_;
  std::unordered_map<int, std::vector<TensorSpan>> modules_;
  std::mutex mu_;
  std::condition_variable cv_consumer_, cv_producer_;
  std::deque<Landing> landings_;
  std::deque<PendingRelease> releases_;
  std::thread thread_;
  std::atomic<bool> running_{false};
  std::atomic<bool> aborted_{false};
  RingStats stats_;
};

}  // namespace bgcore

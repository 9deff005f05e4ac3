// WeightSlotTable: the state machine of one ring of GPU weight slots (one table per module type).
//
// Host-resident weights (experts of a model that does not fit HBM, or whole layers in streamed
// prefill) are copied into a small ring of device slots in *forward order*: the model installs the
// order once ("weight copy queue"), then every forward pass walks it.  A producer thread claims FREE
// slots and fills them; the consumer (the model's forward) leases the slot of the module it needs,
// computes, and releases it — possibly asynchronously, on a stream event.
//
//        claim            landed           acquire            release(async)       reclaim
//   FREE ------> FILLING ------> PRESENT ---------> LEASED ----------------> PENDING_RELEASE ---> FREE
//                                                      \---- release(sync) ----------------------> FREE
//
// Passes: a pass is one walk over the queue.  At most kMaxOpenPasses passes are open; with `carry`
// the producer may run ahead into the next pass as soon as the current one is fully *produced*
// (so the first modules of the next micro-batch are already resident when it starts).
// Skips: modules known to be idle in the current pass (experts no token was routed to) are marked
// and neither produced nor expected by the consumer.  Abort: every pass is cancelled; slots in
// flight return to FREE as they land / are released.
//
// This header is free of CUDA and of threads (callers serialise access), so it is unit-tested on
// its own.  Reference parity: core/GPU_Weight_Buffer/weight_slot_table.h:24-122.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_set>
#include <vector>

namespace bgcore {

enum class SlotState : int { FREE = 0, FILLING = 1, PRESENT = 2, LEASED = 3, PENDING_RELEASE = 4 };

constexpr int kMaxOpenPasses = 2;

struct Slot {
  SlotState state = SlotState::FREE;
  int module = -1;        // index into the queue's module list
  uint64_t pass = 0;      // pass the content belongs to
  bool doomed = false;    // aborted while in flight: goes to FREE instead of PRESENT
};

struct Production {
  int slot = -1;
  int module = -1;
  uint64_t pass = 0;
};

class WeightSlotTable {
 public:
  explicit WeightSlotTable(int num_slots = 0) : slots_(num_slots) {}

  void install_queue(const std::vector<int>& modules) {
    queue_ = modules;
    reset_cursors();
  }
  int num_slots() const { return static_cast<int>(slots_.size()); }
  const Slot& slot(int i) const { return slots_[i]; }
  size_t queue_len() const { return queue_.size(); }
  int open_passes() const { return static_cast<int>(passes_.size()); }
  uint64_t produced_total() const { return produced_total_; }
  uint64_t skipped_total() const { return skipped_total_; }

  // ---- passes
  // Returns the new pass id, or 0 if kMaxOpenPasses are already open.
  uint64_t begin_pass(bool carry) {
    if (static_cast<int>(passes_.size()) >= kMaxOpenPasses) return 0;
    Pass p;
    p.id = ++next_pass_id_;
    p.carry = carry;
    passes_.push_back(p);
    return p.id;
  }
  // The oldest pass is finished by the consumer.  Returns false if it still has unconsumed modules.
  bool end_pass() {
    if (passes_.empty()) return false;
    Pass& p = passes_.front();
    skip_forward_consumer(p);
    if (p.cons_pos < queue_.size()) return false;
    passes_.pop_front();
    return true;
  }
  void skip_modules(const std::vector<int>& modules) {   // applies to the newest open pass
    if (passes_.empty()) return;
    for (int m : modules) passes_.back().skip.insert(m);
  }
  void abort_all() {
    for (auto& s : slots_) {
      if (s.state == SlotState::FILLING || s.state == SlotState::LEASED || s.state == SlotState::PENDING_RELEASE)
        s.doomed = true;
      else if (s.state == SlotState::PRESENT)
        free_slot(s);
    }
    passes_.clear();
  }

  // ---- producer side
  // Next module to copy and the slot to copy it into; false if nothing can be produced now
  // (no FREE slot, no open pass with work left, or running ahead is not allowed).
  bool next_production(Production* out) {
    int free_idx = -1;
    for (int i = 0; i < num_slots(); ++i)
      if (slots_[i].state == SlotState::FREE) { free_idx = i; break; }
    if (free_idx < 0) return false;
    for (size_t pi = 0; pi < passes_.size(); ++pi) {
      Pass& p = passes_[pi];
      while (p.prod_pos < queue_.size() && p.skip.count(queue_[p.prod_pos])) {
        ++p.prod_pos;
        ++skipped_total_;
      }
      if (p.prod_pos < queue_.size()) {
        // a later pass may only be produced when every earlier pass is fully produced and carries
        bool allowed = true;
        for (size_t k = 0; k < pi; ++k)
          if (passes_[k].prod_pos < queue_.size() || !passes_[k].carry) allowed = false;
        if (!allowed) return false;
        Slot& s = slots_[free_idx];
        s.state = SlotState::FILLING;
        s.module = queue_[p.prod_pos];
        s.pass = p.id;
        s.doomed = false;
        out->slot = free_idx;
        out->module = s.module;
        out->pass = p.id;
        ++p.prod_pos;
        ++produced_total_;
        return true;
      }
    }
    return false;
  }
  void landed(int slot_idx) {
    Slot& s = slots_[slot_idx];
    if (s.state != SlotState::FILLING) return;
    if (s.doomed) free_slot(s);
    else s.state = SlotState::PRESENT;
  }

  // ---- consumer side
  // Module the consumer is expected to ask for next in the oldest pass (-1: none).
  int expected_module() {
    if (passes_.empty()) return -1;
    Pass& p = passes_.front();
    skip_forward_consumer(p);
    return p.cons_pos < queue_.size() ? queue_[p.cons_pos] : -1;
  }
  // Lease the slot holding `module` of the oldest pass.  -1: not PRESENT yet; -2: out of order.
  int acquire(int module) {
    if (passes_.empty()) return -2;
    Pass& p = passes_.front();
    skip_forward_consumer(p);
    if (p.cons_pos >= queue_.size() || queue_[p.cons_pos] != module) return -2;
    for (int i = 0; i < num_slots(); ++i) {
      Slot& s = slots_[i];
      if (s.state == SlotState::PRESENT && s.module == module && s.pass == p.id) {
        s.state = SlotState::LEASED;
        ++p.cons_pos;
        return i;
      }
    }
    return -1;
  }
  void release(int slot_idx, bool async) {
    Slot& s = slots_[slot_idx];
    if (s.state != SlotState::LEASED) return;
    if (async) s.state = SlotState::PENDING_RELEASE;
    else free_slot(s);
  }
  void reclaim(int slot_idx) {   // the release event of a PENDING_RELEASE slot completed
    Slot& s = slots_[slot_idx];
    if (s.state == SlotState::PENDING_RELEASE) free_slot(s);
  }

  int count(SlotState st) const {
    int n = 0;
    for (const auto& s : slots_) n += (s.state == st);
    return n;
  }

 private:
  struct Pass {
    uint64_t id = 0;
    bool carry = false;
    size_t prod_pos = 0;
    size_t cons_pos = 0;
    std::unordered_set<int> skip;
  };
  void skip_forward_consumer(Pass& p) {
    while (p.cons_pos < queue_.size() && p.skip.count(queue_[p.cons_pos])) ++p.cons_pos;
  }
  static void free_slot(Slot& s) {
    s.state = SlotState::FREE;
    s.module = -1;
    s.doomed = false;
  }
  void reset_cursors() {
    passes_.clear();
    for (auto& s : slots_) free_slot(s);
  }

  std::vector<Slot> slots_;
  std::vector<int> queue_;
  std::deque<Pass> passes_;
  uint64_t next_pass_id_ = 0;
  uint64_t produced_total_ = 0;
  uint64_t skipped_total_ = 0;
};

}  // namespace bgcore

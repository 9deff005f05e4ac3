// Per-sequence views over the node-shared host KV region for models that do not keep one row per token.
//
// SequencePages: the page list of each sequence in a HostPagedKV region, addressed by *storage* position (the
// index of a stored row inside the sequence's own pages).  Rows are token records: layer l, storage position p
// lives at page[p / page_tokens] + (l * page_tokens + p % page_tokens) * row_bytes.
//
// SlidingWindowView: keeps only the pages that overlap the last `window` raw tokens.  When the raw end passes a
// page boundary far enough, the oldest pages are released; the storage position of raw position r is
// r - (first kept page) * page_tokens.  A write older than the window is refused.  At most window / page + 1 pages
// are held per sequence.
//
// CompressedRatioView<R>: keeps one row per R raw tokens.  The row of raw positions [cR, cR + R) is appended when
// the last of them (raw position with (r + 1) % R == 0) arrives and is stored at position c; other decode steps
// only make sure the capacity for raw_end / R rows exists.  A prefill offload stores raw_len / R rows.
//
// Reference parity: core/KV_Storage/swa_host_paged_kv_worker_view.h (window arithmetic :380-465),
// core/KV_Storage/compressed_ratio_host_paged_kv_worker_view.h (decimation :306-400),
// core/KV_Storage/transformed_host_paged_kv_utils.h.
#pragma once
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "host_kv.h"

namespace bgcore {

class SequencePages {
 public:
  SequencePages(HostPagedKV* kv, int page_tokens, int row_bytes, int layers)
      : kv_(kv), page_tokens_(page_tokens), row_bytes_(row_bytes), layers_(layers) {}
  bool valid() const {
    return kv_ != nullptr && page_tokens_ > 0 && row_bytes_ > 0 && layers_ > 0 &&
           (uint64_t)page_tokens_ * row_bytes_ * layers_ <= kv_->page_bytes();
  }
  // Make the sequence hold at least `pages` pages (all-or-nothing).  false: the region is out of pages.
  bool ensure_pages(int64_t seq, size_t pages);
  // Drop the first `n` pages of the sequence (their rows fall out of every later storage position).
  bool release_prefix(int64_t seq, size_t n);
  void release(int64_t seq);
  size_t num_pages(int64_t seq) const;
  // Address of the row of (layer, storage position); nullptr when the position has no page.
  void* row_ptr(int64_t seq, int layer, size_t storage_pos) const;
  int pages_of(int64_t seq, int32_t* out, int cap) const;
  int page_tokens() const { return page_tokens_; }
  int row_bytes() const { return row_bytes_; }
  HostPagedKV* region() const { return kv_; }

 private:
  HostPagedKV* kv_;
  int page_tokens_, row_bytes_, layers_;
  std::unordered_map<int64_t, std::vector<int32_t>> pages_;
};

struct WindowState {
  size_t start_page = 0;      // raw page index of the first kept page
  size_t max_raw_pos = 0;
  bool has_tokens = false;
};

class SlidingWindowView {
 public:
  SlidingWindowView(HostPagedKV* kv, int page_tokens, int row_bytes, int layers, size_t window_tokens)
      : pages_(kv, page_tokens, row_bytes, layers), window_(window_tokens) {}
  bool valid() const { return pages_.valid() && window_ > 0 && window_ % pages_.page_tokens() == 0; }
  // Advance the sequence to hold raw tokens [.., raw_end).  Returns the number of stored ("active") tokens,
  // -1 when the range is older than the window, -2 when the region has no page left.
  long advance(int64_t seq, size_t raw_end);
  // Storage position of raw position `raw_pos` after advancing to raw_pos + 1 (decode append); same errors.
  long append_position(int64_t seq, size_t raw_pos);
  // Copy `n` rows (raw positions raw_start ..) of one layer into the view; rows older than the window are skipped.
  // Returns rows written or a negative error.
  long write_rows(int64_t seq, int layer, size_t raw_start, const void* rows, size_t n);
  // Copy the rows of the current window (oldest first, at most `cap` rows) out; returns rows copied and the raw
  // position of the first through `first_raw`.
  long read_window(int64_t seq, int layer, void* out, size_t cap, size_t* first_raw) const;
  void release(int64_t seq);
  size_t active_pages(int64_t seq) const { return pages_.num_pages(seq); }
  size_t window_start_token(int64_t seq) const;
  size_t max_pages_per_sequence() const { return window_ / pages_.page_tokens() + 1; }
  SequencePages& pages() { return pages_; }

 private:
  long advance_locked(int64_t seq, size_t raw_end);
  SequencePages pages_;
  size_t window_;
  mutable std::mutex mu_;
  std::unordered_map<int64_t, WindowState> state_;
};

class CompressedRatioView {
 public:
  CompressedRatioView(HostPagedKV* kv, int page_tokens, int row_bytes, int layers, size_t ratio)
      : pages_(kv, page_tokens, row_bytes, layers), ratio_(ratio) {}
  bool valid() const { return pages_.valid() && ratio_ > 0; }
  size_t compressed_tokens(size_t raw_tokens) const { return raw_tokens / ratio_; }
  bool should_append(size_t raw_pos) const { return (raw_pos + 1) % ratio_ == 0; }
  // Prefill offload: `rows` holds raw_len / ratio pooled rows of one layer.  Returns rows stored, -2 out of pages.
  long offload(int64_t seq, int layer, size_t raw_len, const void* rows);
  // Decode step at raw position `raw_pos`: stores `row` at raw_pos / ratio when the position closes a group
  // (returns that storage position), otherwise only reserves capacity (returns -1).  -2: out of pages.
  long append(int64_t seq, int layer, size_t raw_pos, const void* row);
  long read(int64_t seq, int layer, void* out, size_t cap) const;   // stored rows, oldest first
  size_t stored_tokens(int64_t seq) const;
  void release(int64_t seq);
  SequencePages& pages() { return pages_; }

 private:
  bool ensure_locked(int64_t seq, size_t exposed_tokens);
  SequencePages pages_;
  size_t ratio_;
  mutable std::mutex mu_;
  std::unordered_map<int64_t, size_t> exposed_;
};

}  // namespace bgcore

#include "host_kv_views.h"

#include <algorithm>
#include <cstring>

namespace bgcore {

// ---------------------------------------------------------------- SequencePages
bool SequencePages::ensure_pages(int64_t seq, size_t pages) {
  auto& v = pages_[seq];
  if (v.size() >= pages) return true;
  const int need = (int)(pages - v.size());
  std::vector<int32_t> got(need);
  if (!kv_->alloc(need, got.data())) return false;
  v.insert(v.end(), got.begin(), got.end());
  return true;
}

bool SequencePages::release_prefix(int64_t seq, size_t n) {
  auto it = pages_.find(seq);
  if (it == pages_.end() || it->second.size() < n) return false;
  if (n == 0) return true;
  kv_->free_pages(it->second.data(), (int)n);
  it->second.erase(it->second.begin(), it->second.begin() + n);
  return true;
}

void SequencePages::release(int64_t seq) {
  auto it = pages_.find(seq);
  if (it == pages_.end()) return;
  if (!it->second.empty()) kv_->free_pages(it->second.data(), (int)it->second.size());
  pages_.erase(it);
}

size_t SequencePages::num_pages(int64_t seq) const {
  auto it = pages_.find(seq);
  return it == pages_.end() ? 0 : it->second.size();
}

void* SequencePages::row_ptr(int64_t seq, int layer, size_t storage_pos) const {
  auto it = pages_.find(seq);
  if (it == pages_.end() || layer < 0 || layer >= layers_) return nullptr;
  const size_t page = storage_pos / page_tokens_;
  if (page >= it->second.size()) return nullptr;
  auto* base = static_cast<uint8_t*>(kv_->page_ptr(it->second[page]));
  if (base == nullptr) return nullptr;
  return base + ((size_t)layer * page_tokens_ + storage_pos % page_tokens_) * row_bytes_;
}

int SequencePages::pages_of(int64_t seq, int32_t* out, int cap) const {
  auto it = pages_.find(seq);
  if (it == pages_.end()) return 0;
  const int n = std::min<int>(cap, (int)it->second.size());
  std::copy(it->second.begin(), it->second.begin() + n, out);
  return (int)it->second.size();
}

// ---------------------------------------------------------------- SlidingWindowView
long SlidingWindowView::advance_locked(int64_t seq, size_t raw_end) {
  if (raw_end == 0) return 0;
  const size_t pt = pages_.page_tokens();
  const size_t first_needed = raw_end > window_ ? raw_end - window_ : 0;
  const size_t start_page = first_needed / pt;
  const size_t active = raw_end - start_page * pt;
  const size_t need_pages = (active + pt - 1) / pt;
  auto& st = state_[seq];
  if (st.has_tokens && start_page < st.start_page) return -1;           // older than what is kept
  if (st.has_tokens && start_page > st.start_page) {
    const size_t drop = std::min(start_page - st.start_page, pages_.num_pages(seq));
    pages_.release_prefix(seq, drop);
  }
  st.start_page = start_page;
  if (!pages_.ensure_pages(seq, need_pages)) return -2;
  st.max_raw_pos = std::max(st.max_raw_pos, raw_end - 1);
  st.has_tokens = true;
  return (long)active;
}

long SlidingWindowView::advance(int64_t seq, size_t raw_end) {
  std::lock_guard<std::mutex> g(mu_);
  return advance_locked(seq, raw_end);
}

long SlidingWindowView::append_position(int64_t seq, size_t raw_pos) {
  std::lock_guard<std::mutex> g(mu_);
  const long active = advance_locked(seq, raw_pos + 1);
  return active < 0 ? active : active - 1;
}

long SlidingWindowView::write_rows(int64_t seq, int layer, size_t raw_start, const void* rows, size_t n) {
  std::lock_guard<std::mutex> g(mu_);
  if (n == 0) return 0;
  const long active = advance_locked(seq, raw_start + n);
  if (active < 0) return active;
  const size_t start_tok = state_[seq].start_page * pages_.page_tokens();
  const size_t rb = pages_.row_bytes();
  long written = 0;
  for (size_t i = 0; i < n; ++i) {
    const size_t raw = raw_start + i;
    if (raw < start_tok) continue;                                       // already outside the window
    void* dst = pages_.row_ptr(seq, layer, raw - start_tok);
    if (dst == nullptr) return -3;
    std::memcpy(dst, static_cast<const uint8_t*>(rows) + i * rb, rb);
    ++written;
  }
  return written;
}

long SlidingWindowView::read_window(int64_t seq, int layer, void* out, size_t cap, size_t* first_raw) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = state_.find(seq);
  if (it == state_.end() || !it->second.has_tokens) return 0;
  const size_t pt = pages_.page_tokens();
  const size_t end = it->second.max_raw_pos + 1;
  const size_t start_tok = it->second.start_page * pt;
  size_t first = end > window_ ? end - window_ : 0;
  if (end - first > cap) first = end - cap;
  const size_t rb = pages_.row_bytes();
  for (size_t raw = first; raw < end; ++raw) {
    const void* src = pages_.row_ptr(seq, layer, raw - start_tok);
    if (src == nullptr) return -3;
    std::memcpy(static_cast<uint8_t*>(out) + (raw - first) * rb, src, rb);
  }
  if (first_raw != nullptr) *first_raw = first;
  return (long)(end - first);
}

void SlidingWindowView::release(int64_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  pages_.release(seq);
  state_.erase(seq);
}

size_t SlidingWindowView::window_start_token(int64_t seq) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = state_.find(seq);
  return it == state_.end() ? 0 : it->second.start_page * pages_.page_tokens();
}

// ---------------------------------------------------------------- CompressedRatioView
bool CompressedRatioView::ensure_locked(int64_t seq, size_t exposed_tokens) {
  const size_t pt = pages_.page_tokens();
  const size_t cap_tokens = std::max<size_t>(1, exposed_tokens);
  if (!pages_.ensure_pages(seq, (cap_tokens + pt - 1) / pt)) return false;
  auto& e = exposed_[seq];
  e = std::max(e, exposed_tokens);
  return true;
}

long CompressedRatioView::offload(int64_t seq, int layer, size_t raw_len, const void* rows) {
  std::lock_guard<std::mutex> g(mu_);
  const size_t n = compressed_tokens(raw_len);
  if (!ensure_locked(seq, n)) return -2;
  const size_t rb = pages_.row_bytes();
  for (size_t c = 0; c < n; ++c) {
    void* dst = pages_.row_ptr(seq, layer, c);
    if (dst == nullptr) return -3;
    std::memcpy(dst, static_cast<const uint8_t*>(rows) + c * rb, rb);
  }
  return (long)n;
}

long CompressedRatioView::append(int64_t seq, int layer, size_t raw_pos, const void* row) {
  std::lock_guard<std::mutex> g(mu_);
  if (!should_append(raw_pos)) {
    if (!ensure_locked(seq, compressed_tokens(raw_pos + 1))) return -2;
    return -1;
  }
  const size_t c = raw_pos / ratio_;
  if (!ensure_locked(seq, c + 1)) return -2;
  void* dst = pages_.row_ptr(seq, layer, c);
  if (dst == nullptr) return -3;
  std::memcpy(dst, row, pages_.row_bytes());
  return (long)c;
}

long CompressedRatioView::read(int64_t seq, int layer, void* out, size_t cap) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = exposed_.find(seq);
  if (it == exposed_.end()) return 0;
  const size_t n = std::min(cap, it->second);
  const size_t rb = pages_.row_bytes();
  for (size_t c = 0; c < n; ++c) {
    const void* src = pages_.row_ptr(seq, layer, c);
    if (src == nullptr) return -3;
    std::memcpy(static_cast<uint8_t*>(out) + c * rb, src, rb);
  }
  return (long)n;
}

size_t CompressedRatioView::stored_tokens(int64_t seq) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = exposed_.find(seq);
  return it == exposed_.end() ? 0 : it->second;
}

void CompressedRatioView::release(int64_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  pages_.release(seq);
  exposed_.erase(seq);
}

}  // namespace bgcore

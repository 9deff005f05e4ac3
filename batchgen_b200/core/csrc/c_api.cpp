// C ABI of the native engine (loaded from Python with ctypes: batchgen_b200/core/native.py).
// The reference exposes the same objects through pybind11 (core/batchgen_Binding.cpp:616-1262).
#include <cstring>
#include <vector>

#include "host_kv.h"
#include "host_kv_views.h"
#include "weight_daemon.h"
#include "weight_ring.h"

using namespace bgcore;

extern "C" {

// ------------------------------------------------------------------ weight ring
// backend: 0 = host (memcpy), 1 = CUDA on `device`.  Returns nullptr if the CUDA backend is unusable.
void* bgc_ring_create(int num_slots, unsigned long long slot_bytes, int backend, int device) {
  std::unique_ptr<CopyBackend> be = backend == 1 ? make_cuda_backend(device) : make_host_backend();
  if (!be) return nullptr;
  return new WeightRing(num_slots, slot_bytes, std::move(be));
}
void bgc_ring_destroy(void* r) { delete static_cast<WeightRing*>(r); }

// tensors of the module: host pointers + sizes; slot offsets are returned through `offsets`.
int bgc_ring_register_module(void* r, int module, const void* const* ptrs, const unsigned long long* sizes, int n,
                             unsigned long long* offsets) {
  std::vector<TensorSpan> spans(n);
  for (int i = 0; i < n; ++i) spans[i] = TensorSpan{ptrs[i], static_cast<size_t>(sizes[i]), 0};
  if (!static_cast<WeightRing*>(r)->register_module(module, &spans)) return -1;
  for (int i = 0; i < n; ++i) offsets[i] = spans[i].slot_offset;
  return 0;
}
void bgc_ring_install_queue(void* r, const int* modules, int n) {
  static_cast<WeightRing*>(r)->install_queue(std::vector<int>(modules, modules + n));
}
unsigned long long bgc_ring_begin_pass(void* r, int carry) { return static_cast<WeightRing*>(r)->begin_pass(carry != 0); }
int bgc_ring_end_pass(void* r) { return static_cast<WeightRing*>(r)->end_pass() ? 0 : -1; }
void bgc_ring_skip(void* r, const int* modules, int n) {
  static_cast<WeightRing*>(r)->skip_modules(std::vector<int>(modules, modules + n));
}
void bgc_ring_abort(void* r) { static_cast<WeightRing*>(r)->abort_passes(); }
void bgc_ring_start(void* r) { static_cast<WeightRing*>(r)->start_producer(); }
void bgc_ring_stop(void* r) { static_cast<WeightRing*>(r)->stop_producer(); }
void* bgc_ring_get(void* r, int module, int timeout_ms, int* slot_out) {
  return static_cast<WeightRing*>(r)->get_weights(module, timeout_ms, slot_out);
}
void bgc_ring_release(void* r, int slot, void* stream) { static_cast<WeightRing*>(r)->release(slot, stream); }
int bgc_ring_count_state(void* r, int state) { return static_cast<WeightRing*>(r)->count_state(state); }
// out: modules_copied, modules_skipped, bytes_copied, get_calls, get_wait_us, stalls, copy_us
void bgc_ring_stats(void* r, unsigned long long* out) {
  RingStats s = static_cast<WeightRing*>(r)->stats();
  out[0] = s.modules_copied; out[1] = s.modules_skipped; out[2] = s.bytes_copied; out[3] = s.get_calls;
  out[4] = s.get_wait_us; out[5] = s.stalls; out[6] = static_cast<unsigned long long>(s.copy_seconds * 1e6);
}

// ------------------------------------------------------------------ host paged KV + prefix coordinator
void* bgc_hostkv_create(unsigned long long num_pages, unsigned long long page_bytes, unsigned long long prefix_slots,
                        int* fd_out) {
  auto* h = new HostPagedKV();
  int fd = h->create(num_pages, page_bytes, prefix_slots);
  if (fd < 0) {
    delete h;
    return nullptr;
  }
  if (fd_out) *fd_out = fd;
  return h;
}
void* bgc_hostkv_attach(int fd) {
  auto* h = new HostPagedKV();
  if (!h->attach(fd)) {
    delete h;
    return nullptr;
  }
  return h;
}
void bgc_hostkv_destroy(void* h) { delete static_cast<HostPagedKV*>(h); }
int bgc_hostkv_alloc(void* h, int n, int* out) { return static_cast<HostPagedKV*>(h)->alloc(n, out) ? 0 : -1; }
void bgc_hostkv_share(void* h, const int* pages, int n) { static_cast<HostPagedKV*>(h)->share(pages, n); }
void bgc_hostkv_free(void* h, const int* pages, int n) { static_cast<HostPagedKV*>(h)->free_pages(pages, n); }
int bgc_hostkv_refcount(void* h, int page) { return static_cast<HostPagedKV*>(h)->refcount(page); }
unsigned long long bgc_hostkv_num_free(void* h) { return static_cast<HostPagedKV*>(h)->num_free(); }
unsigned long long bgc_hostkv_num_pages(void* h) { return static_cast<HostPagedKV*>(h)->num_pages(); }
void* bgc_hostkv_page_ptr(void* h, int page) { return static_cast<HostPagedKV*>(h)->page_ptr(page); }
void* bgc_hostkv_base(void* h) { return static_cast<HostPagedKV*>(h)->base(); }
unsigned long long bgc_hostkv_bytes(void* h) { return static_cast<HostPagedKV*>(h)->mapped_bytes(); }
int bgc_hostkv_audit(void* h) { return static_cast<HostPagedKV*>(h)->audit(); }
int bgc_prefix_commit(void* h, const unsigned char* keys, const int* pages, int n) {
  return static_cast<HostPagedKV*>(h)->prefix_commit(keys, pages, n);
}
int bgc_prefix_lookup_attach(void* h, const unsigned char* keys, int n, int* pages_out) {
  return static_cast<HostPagedKV*>(h)->prefix_lookup_attach(keys, n, pages_out);
}
int bgc_prefix_evict(void* h, int want) { return static_cast<HostPagedKV*>(h)->prefix_evict(want); }
int bgc_prefix_clear(void* h) { return static_cast<HostPagedKV*>(h)->prefix_clear(); }
void bgc_prefix_stats(void* h, unsigned long long* out) {
  uint64_t s[4];
  static_cast<HostPagedKV*>(h)->prefix_stats(s);
  for (int i = 0; i < 4; ++i) out[i] = s[i];
}


// ------------------------------------------------------------------ sliding-window / compressed-ratio host views
void* bgc_swa_create(void* hostkv, int page_tokens, int row_bytes, int layers, unsigned long long window_tokens) {
  auto* v = new SlidingWindowView(static_cast<HostPagedKV*>(hostkv), page_tokens, row_bytes, layers, window_tokens);
  if (!v->valid()) {
    delete v;
    return nullptr;
  }
  return v;
}
void bgc_swa_destroy(void* v) { delete static_cast<SlidingWindowView*>(v); }
long bgc_swa_advance(void* v, long long seq, unsigned long long raw_end) {
  return static_cast<SlidingWindowView*>(v)->advance(seq, raw_end);
}
long bgc_swa_append_position(void* v, long long seq, unsigned long long raw_pos) {
  return static_cast<SlidingWindowView*>(v)->append_position(seq, raw_pos);
}
long bgc_swa_write_rows(void* v, long long seq, int layer, unsigned long long raw_start, const void* rows,
                        unsigned long long n) {
  return static_cast<SlidingWindowView*>(v)->write_rows(seq, layer, raw_start, rows, n);
}
long bgc_swa_read_window(void* v, long long seq, int layer, void* out, unsigned long long cap,
                         unsigned long long* first_raw) {
  size_t first = 0;
  const long n = static_cast<SlidingWindowView*>(v)->read_window(seq, layer, out, cap, &first);
  if (first_raw != nullptr) *first_raw = first;
  return n;
}
void bgc_swa_release(void* v, long long seq) { static_cast<SlidingWindowView*>(v)->release(seq); }
unsigned long long bgc_swa_active_pages(void* v, long long seq) {
  return static_cast<SlidingWindowView*>(v)->active_pages(seq);
}
unsigned long long bgc_swa_window_start(void* v, long long seq) {
  return static_cast<SlidingWindowView*>(v)->window_start_token(seq);
}

void* bgc_cratio_create(void* hostkv, int page_tokens, int row_bytes, int layers, unsigned long long ratio) {
  auto* v = new CompressedRatioView(static_cast<HostPagedKV*>(hostkv), page_tokens, row_bytes, layers, ratio);
  if (!v->valid()) {
    delete v;
    return nullptr;
  }
  return v;
}
void bgc_cratio_destroy(void* v) { delete static_cast<CompressedRatioView*>(v); }
long bgc_cratio_offload(void* v, long long seq, int layer, unsigned long long raw_len, const void* rows) {
  return static_cast<CompressedRatioView*>(v)->offload(seq, layer, raw_len, rows);
}
long bgc_cratio_append(void* v, long long seq, int layer, unsigned long long raw_pos, const void* row) {
  return static_cast<CompressedRatioView*>(v)->append(seq, layer, raw_pos, row);
}
long bgc_cratio_read(void* v, long long seq, int layer, void* out, unsigned long long cap) {
  return static_cast<CompressedRatioView*>(v)->read(seq, layer, out, cap);
}
unsigned long long bgc_cratio_stored(void* v, long long seq) {
  return static_cast<CompressedRatioView*>(v)->stored_tokens(seq);
}
unsigned long long bgc_cratio_pages(void* v, long long seq) {
  return static_cast<CompressedRatioView*>(v)->pages().num_pages(seq);
}
void bgc_cratio_release(void* v, long long seq) { static_cast<CompressedRatioView*>(v)->release(seq); }


// ------------------------------------------------------------------ node weight daemon
// peers: "node=host:port,node=host:port"
void* bgc_wd_create(int node, const char* socket_path, int listen_port, const char* peers, int staging_slots,
                    unsigned long long slot_bytes, int prefetch_depth, int acquire_wait_ms) {
  DaemonConfig c;
  c.node = node;
  c.socket_path = socket_path ? socket_path : "";
  c.listen_port = listen_port;
  c.staging_slots = staging_slots;
  c.slot_bytes = slot_bytes;
  c.prefetch_depth = prefetch_depth;
  c.acquire_wait_ms = acquire_wait_ms;
  std::string p = peers ? peers : "";
  size_t pos = 0;
  while (pos < p.size()) {
    size_t end = p.find(',', pos);
    if (end == std::string::npos) end = p.size();
    const std::string item = p.substr(pos, end - pos);
    const size_t eq = item.find('=');
    if (eq != std::string::npos) c.peers[std::atoi(item.substr(0, eq).c_str())] = item.substr(eq + 1);
    pos = end + 1;
  }
  return new WeightDaemon(c);
}
void bgc_wd_destroy(void* d) { delete static_cast<WeightDaemon*>(d); }
void bgc_wd_set_store(void* d, const void* base, unsigned long long bytes) {
  static_cast<WeightDaemon*>(d)->set_local_store(base, bytes);
}
int bgc_wd_add_module(void* d, const char* key, int owner, unsigned long long offset, unsigned long long bytes) {
  return static_cast<WeightDaemon*>(d)->add_module(key, owner, offset, bytes) ? 0 : -1;
}
// keys: newline-separated
void bgc_wd_set_schedule(void* d, const char* keys) {
  std::vector<std::string> v;
  std::string s = keys ? keys : "";
  size_t pos = 0;
  while (pos < s.size()) {
    size_t end = s.find('\n', pos);
    if (end == std::string::npos) end = s.size();
    if (end > pos) v.push_back(s.substr(pos, end - pos));
    pos = end + 1;
  }
  static_cast<WeightDaemon*>(d)->set_schedule(v);
}
int bgc_wd_start(void* d) { return static_cast<WeightDaemon*>(d)->start() ? 0 : -1; }
void bgc_wd_stop(void* d) { static_cast<WeightDaemon*>(d)->stop(); }
int bgc_wd_staging_fd(void* d) { return static_cast<WeightDaemon*>(d)->staging_fd(); }
unsigned long long bgc_wd_staging_bytes(void* d) { return static_cast<WeightDaemon*>(d)->staging_bytes(); }
unsigned long long bgc_wd_epoch(void* d) { return static_cast<WeightDaemon*>(d)->epoch(); }
unsigned long long bgc_wd_begin_swap(void* d) { return static_cast<WeightDaemon*>(d)->begin_swap(); }
static int copy_out(const std::string& s, char* out, int cap) {
  const int n = (int)std::min<size_t>(s.size(), cap > 0 ? cap - 1 : 0);
  if (cap > 0) {
    std::memcpy(out, s.data(), n);
    out[n] = 0;
  }
  return (int)s.size();
}
int bgc_wd_finish_swap(void* d, char* out, int cap) { return copy_out(static_cast<WeightDaemon*>(d)->finish_swap(), out, cap); }
int bgc_wd_status(void* d, char* out, int cap) { return copy_out(static_cast<WeightDaemon*>(d)->status(), out, cap); }

void* bgc_wdc_create() { return new DaemonClient(); }
void bgc_wdc_destroy(void* c) { delete static_cast<DaemonClient*>(c); }
int bgc_wdc_connect(void* c, const char* path) { return static_cast<DaemonClient*>(c)->connect_to(path) ? 0 : -1; }
int bgc_wdc_hello(void* c, unsigned worker, unsigned long long epoch) { return static_cast<DaemonClient*>(c)->hello(worker, epoch); }
int bgc_wdc_acquire(void* c, const char* key, int timeout_ms, int* slot, unsigned long long* offset,
                    unsigned long long* bytes) {
  uint64_t off = 0, by = 0;
  const int rc = static_cast<DaemonClient*>(c)->acquire(key, timeout_ms, slot, &off, &by);
  *offset = off;
  *bytes = by;
  return rc;
}
int bgc_wdc_release(void* c, const char* key) { return static_cast<DaemonClient*>(c)->release(key); }
void bgc_wdc_close(void* c) { static_cast<DaemonClient*>(c)->close_conn(); }
int bgc_wdc_error(void* c, char* out, int cap) { return copy_out(static_cast<DaemonClient*>(c)->last_error(), out, cap); }

}  // extern "C"

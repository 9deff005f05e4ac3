// Node-shared paged host KV region and the prefix-cache coordinator that lives inside it.
//
// HostPagedKV: one anonymous shared-memory file (memfd) holds a control block followed by
// `num_pages` pages of `page_bytes`.  The server creates it and hands the fd to every worker; each
// worker attaches (mmap) and, on a GPU box, pins the mapping so that pages can be the source or target
// of asynchronous copies.  The control block carries a process-shared mutex, a free stack and a
// reference count per page, so that any process can allocate, share (prefix reuse) and free pages.
//
// PrefixCoordinator: an open-addressing hash table in the same region keyed by a 256-bit hash chain
// over page-sized blocks of token ids (key_i = H(key_{i-1} || block_i)).  commit() publishes the pages
// of a prefilled prefix (the cache takes a reference on each), lookup_and_attach() returns the longest
// cached chain and takes a reference per page for the caller, evict() drops least-recently-used leaf
// entries whose page only the cache still references, clear() drops everything.
//
// Reference parity: core/KV_Storage/host_paged_kv_manager.h, host_paged_kv_backend.{h,cpp},
// host_kv_page_table.{h,cpp} (node-shared paged region, allocator, stats/audit) and
// core/KV_Storage/host_prefix_cache_coordinator.h:13-174 (commit / lookup_and_attach / evict / clear).
#pragma once
#include <pthread.h>

#include <cstddef>
#include <cstdint>
#include <vector>

namespace bgcore {

constexpr uint64_t kHostKvMagic = 0x42474b5648303031ull;   // "BGKVH001"

struct PrefixEntry {
  uint8_t key[32];
  int32_t page;          // -1: empty, -2: tombstone
  int32_t parent;        // table index of the parent entry or -1
  int32_t children;
  uint32_t pad;
  uint64_t tick;         // last use
};

struct HostKvControl {
  uint64_t magic;
  uint64_t num_pages;
  uint64_t page_bytes;
  uint64_t pages_offset;      // byte offset of page 0 from the mapping base
  uint64_t table_slots;       // prefix table capacity
  uint64_t table_offset;
  uint64_t free_top;          // number of entries in the free stack
  uint64_t clock;
  uint64_t prefix_entries, prefix_hits, prefix_misses, prefix_evicted;
  pthread_mutex_t mu;
  // followed by: int32 free_stack[num_pages]; int32 refcnt[num_pages]
};

class HostPagedKV {
 public:
  HostPagedKV() {}
  ~HostPagedKV();
  // Create a new region (returns its fd, -1 on failure) or attach to an existing one.
  int create(uint64_t num_pages, uint64_t page_bytes, uint64_t prefix_slots);
  bool attach(int fd);
  void detach();

  bool alloc(int n, int32_t* out);           // all-or-nothing
  void share(const int32_t* pages, int n);
  void free_pages(const int32_t* pages, int n);
  int refcount(int32_t page);
  uint64_t num_free();
  uint64_t num_pages() const { return ctl_ ? ctl_->num_pages : 0; }
  uint64_t page_bytes() const { return ctl_ ? ctl_->page_bytes : 0; }
  void* page_ptr(int32_t page) const;
  void* base() const { return base_; }
  size_t mapped_bytes() const { return bytes_; }
  int fd() const { return fd_; }
  // Audit: every page is either on the free stack (refcount 0) or referenced; returns the number of
  // inconsistencies found.
  int audit();

  // ---- prefix coordinator
  int prefix_commit(const uint8_t* keys, const int32_t* pages, int n);              // -> new entries
  int prefix_lookup_attach(const uint8_t* keys, int n, int32_t* pages_out);         // -> matched length
  int prefix_evict(int want_pages);                                                  // -> pages freed
  int prefix_clear();
  void prefix_stats(uint64_t out[4]);                                                // entries, hits, misses, evicted

 private:
  struct Lock;
  int32_t* free_stack() const;
  int32_t* refcnt() const;
  PrefixEntry* table() const;
  int64_t find(const uint8_t* key) const;
  void release_locked(int32_t page);

  void* base_ = nullptr;
  size_t bytes_ = 0;
  int fd_ = -1;
  bool owner_ = false;
  HostKvControl* ctl_ = nullptr;
};

}  // namespace bgcore

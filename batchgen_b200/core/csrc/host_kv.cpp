// HostPagedKV + prefix coordinator implementation.  See host_kv.h.
#include "host_kv.h"

#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

namespace bgcore {

struct HostPagedKV::Lock {
  pthread_mutex_t* m;
  explicit Lock(pthread_mutex_t* mu) : m(mu) {
    int rc = pthread_mutex_lock(m);
    if (rc == EOWNERDEAD) pthread_mutex_consistent(m);   // a process died holding the lock: state is re-audited
  }
  ~Lock() { pthread_mutex_unlock(m); }
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

HostPagedKV::~HostPagedKV() { detach(); }

int32_t* HostPagedKV::free_stack() const {
  return reinterpret_cast<int32_t*>(static_cast<char*>(base_) + align_up(sizeof(HostKvControl), 64));
}
int32_t* HostPagedKV::refcnt() const { return free_stack() + ctl_->num_pages; }
PrefixEntry* HostPagedKV::table() const {
  return reinterpret_cast<PrefixEntry*>(static_cast<char*>(base_) + ctl_->table_offset);
}
void* HostPagedKV::page_ptr(int32_t page) const {
  return static_cast<char*>(base_) + ctl_->pages_offset + static_cast<size_t>(page) * ctl_->page_bytes;
}

int HostPagedKV::create(uint64_t num_pages, uint64_t page_bytes, uint64_t prefix_slots) {
  size_t head = align_up(sizeof(HostKvControl), 64) + 2 * num_pages * sizeof(int32_t);
  size_t table_off = align_up(head, 64);
  size_t pages_off = align_up(table_off + prefix_slots * sizeof(PrefixEntry), 4096);
  size_t total = pages_off + num_pages * page_bytes;
  int fd = static_cast<int>(syscall(SYS_memfd_create, "bg_host_kv", 0));
  if (fd < 0) return -1;
  if (ftruncate(fd, static_cast<off_t>(total)) != 0) {
    close(fd);
    return -1;
  }
  void* p = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    close(fd);
    return -1;
  }
  base_ = p;
  bytes_ = total;
  fd_ = fd;
  owner_ = true;
  ctl_ = static_cast<HostKvControl*>(p);
  std::memset(ctl_, 0, sizeof(HostKvControl));
  ctl_->num_pages = num_pages;
  ctl_->page_bytes = page_bytes;
  ctl_->pages_offset = pages_off;
  ctl_->table_slots = prefix_slots;
  ctl_->table_offset = table_off;
  pthread_mutexattr_t at;
  pthread_mutexattr_init(&at);
  pthread_mutexattr_setpshared(&at, PTHREAD_PROCESS_SHARED);
  pthread_mutexattr_setrobust(&at, PTHREAD_MUTEX_ROBUST);
  pthread_mutex_init(&ctl_->mu, &at);
  pthread_mutexattr_destroy(&at);
  int32_t* fs = free_stack();
  for (uint64_t i = 0; i < num_pages; ++i) fs[i] = static_cast<int32_t>(num_pages - 1 - i);
  ctl_->free_top = num_pages;
  std::memset(refcnt(), 0, num_pages * sizeof(int32_t));
  PrefixEntry* t = table();
  for (uint64_t i = 0; i < prefix_slots; ++i) {
    t[i].page = -1;
    t[i].parent = -1;
    t[i].children = 0;
    t[i].tick = 0;
  }
  ctl_->magic = kHostKvMagic;
  return fd;
}

bool HostPagedKV::attach(int fd) {
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < static_cast<off_t>(sizeof(HostKvControl))) return false;
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) return false;
  if (static_cast<HostKvControl*>(p)->magic != kHostKvMagic) {
    munmap(p, static_cast<size_t>(st.st_size));
    return false;
  }
  base_ = p;
  bytes_ = static_cast<size_t>(st.st_size);
  fd_ = fd;
  owner_ = false;
  ctl_ = static_cast<HostKvControl*>(p);
  return true;
}

void HostPagedKV::detach() {
  if (base_ != nullptr) munmap(base_, bytes_);
  if (owner_ && fd_ >= 0) close(fd_);
  base_ = nullptr;
  ctl_ = nullptr;
  fd_ = -1;
}

bool HostPagedKV::alloc(int n, int32_t* out) {
  Lock l(&ctl_->mu);
  if (static_cast<uint64_t>(n) > ctl_->free_top) return false;
  int32_t* fs = free_stack();
  int32_t* rc = refcnt();
  for (int i = 0; i < n; ++i) {
    int32_t p = fs[--ctl_->free_top];
    rc[p] = 1;
    out[i] = p;
  }
  return true;
}

void HostPagedKV::share(const int32_t* pages, int n) {
  Lock l(&ctl_->mu);
  int32_t* rc = refcnt();
  for (int i = 0; i < n; ++i)
    if (rc[pages[i]] > 0) rc[pages[i]] += 1;
}

void HostPagedKV::release_locked(int32_t page) {
  int32_t* rc = refcnt();
  if (rc[page] <= 0) return;
  if (--rc[page] == 0) free_stack()[ctl_->free_top++] = page;
}

void HostPagedKV::free_pages(const int32_t* pages, int n) {
  Lock l(&ctl_->mu);
  for (int i = 0; i < n; ++i) release_locked(pages[i]);
}

int HostPagedKV::refcount(int32_t page) {
  Lock l(&ctl_->mu);
  return refcnt()[page];
}

uint64_t HostPagedKV::num_free() {
  Lock l(&ctl_->mu);
  return ctl_->free_top;
}

int HostPagedKV::audit() {
  Lock l(&ctl_->mu);
  std::vector<char> on_stack(ctl_->num_pages, 0);
  int bad = 0;
  int32_t* fs = free_stack();
  int32_t* rc = refcnt();
  for (uint64_t i = 0; i < ctl_->free_top; ++i) {
    int32_t p = fs[i];
    if (p < 0 || static_cast<uint64_t>(p) >= ctl_->num_pages || on_stack[p]) { ++bad; continue; }
    on_stack[p] = 1;
    if (rc[p] != 0) ++bad;
  }
  for (uint64_t p = 0; p < ctl_->num_pages; ++p)
    if (!on_stack[p] && rc[p] <= 0) ++bad;
  return bad;
}

// ------------------------------------------------------------------ prefix coordinator
static uint64_t key_hash(const uint8_t* key) {
  uint64_t h;
  std::memcpy(&h, key, 8);
  return h * 0x9E3779B97F4A7C15ull;
}

int64_t HostPagedKV::find(const uint8_t* key) const {
  const uint64_t n = ctl_->table_slots;
  if (n == 0) return -1;
  PrefixEntry* t = table();
  uint64_t i = key_hash(key) % n;
  for (uint64_t probe = 0; probe < n; ++probe, i = (i + 1) % n) {
    if (t[i].page == -1) return -1;
    if (t[i].page >= 0 && std::memcmp(t[i].key, key, 32) == 0) return static_cast<int64_t>(i);
  }
  return -1;
}

int HostPagedKV::prefix_commit(const uint8_t* keys, const int32_t* pages, int n) {
  Lock l(&ctl_->mu);
  const uint64_t cap = ctl_->table_slots;
  PrefixEntry* t = table();
  int added = 0;
  int64_t parent = -1;
  for (int k = 0; k < n; ++k) {
    const uint8_t* key = keys + 32 * k;
    int64_t idx = find(key);
    if (idx < 0) {
      if (cap == 0 || ctl_->prefix_entries * 10 >= cap * 7) break;   // keep the load factor below 0.7
      uint64_t i = key_hash(key) % cap;
      while (t[i].page >= 0) i = (i + 1) % cap;
      std::memcpy(t[i].key, key, 32);
      t[i].page = pages[k];
      t[i].parent = static_cast<int32_t>(parent);
      t[i].children = 0;
      if (parent >= 0) t[parent].children += 1;
      refcnt()[pages[k]] += 1;          // the cache's own reference
      ctl_->prefix_entries += 1;
      idx = static_cast<int64_t>(i);
      ++added;
    }
    t[idx].tick = ++ctl_->clock;
    parent = idx;
  }
  return added;
}

int HostPagedKV::prefix_lookup_attach(const uint8_t* keys, int n, int32_t* pages_out) {
  Lock l(&ctl_->mu);
  PrefixEntry* t = table();
  int m = 0;
  for (; m < n; ++m) {
    int64_t idx = find(keys + 32 * m);
    if (idx < 0) break;
    t[idx].tick = ++ctl_->clock;
    pages_out[m] = t[idx].page;
    refcnt()[t[idx].page] += 1;         // reference for the caller
  }
  if (m > 0) ctl_->prefix_hits += 1;
  else ctl_->prefix_misses += 1;
  return m;
}

int HostPagedKV::prefix_evict(int want_pages) {
  Lock l(&ctl_->mu);
  PrefixEntry* t = table();
  int freed = 0;
  while (freed < want_pages) {
    int64_t best = -1;
    for (uint64_t i = 0; i < ctl_->table_slots; ++i) {
      if (t[i].page < 0 || t[i].children != 0 || refcnt()[t[i].page] != 1) continue;
      if (best < 0 || t[i].tick < t[best].tick) best = static_cast<int64_t>(i);
    }
    if (best < 0) break;
    if (t[best].parent >= 0) t[t[best].parent].children -= 1;
    release_locked(t[best].page);
    t[best].page = -2;                  // tombstone keeps probe chains intact
    ctl_->prefix_entries -= 1;
    ctl_->prefix_evicted += 1;
    ++freed;
  }
  return freed;
}

int HostPagedKV::prefix_clear() {
  Lock l(&ctl_->mu);
  PrefixEntry* t = table();
  int n = 0;
  for (uint64_t i = 0; i < ctl_->table_slots; ++i) {
    if (t[i].page >= 0) {
      release_locked(t[i].page);
      ++n;
    }
    t[i].page = -1;
    t[i].parent = -1;
    t[i].children = 0;
  }
  ctl_->prefix_entries = 0;
  return n;
}

void HostPagedKV::prefix_stats(uint64_t out[4]) {
  Lock l(&ctl_->mu);
  out[0] = ctl_->prefix_entries;
  out[1] = ctl_->prefix_hits;
  out[2] = ctl_->prefix_misses;
  out[3] = ctl_->prefix_evicted;
}

}  // namespace bgcore

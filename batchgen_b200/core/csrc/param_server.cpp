// Parameter server and replica control block (host side, no CUDA).
//
// ParameterStore: the server process allocates ONE anonymous shared region (memfd) for all weights of the
// node, reads converted checkpoint shards (raw tensor bytes back to back) into it with parallel pread
// threads, and hands the descriptor to the workers, which map it (and pin it for DMA) instead of each
// holding a private copy.  Huge pages are requested with madvise when available.
//
// ReplicaControlBlock: a small shared-memory block of atomics through which the ranks of a weight replica
// group coordinate a streamed pass: per-(member, module type) barrier words A (slot published by its owner)
// and B (every reader has pulled, the owner may reuse the slot), per-slot publication sequence numbers,
// and abort flags.  All waits are bounded by a timeout.
//
// Reference parity: core/Parameter_Server/Parameter_Server.{h,cpp} + posix_shm.{h,cpp} (memfd allocation,
// checkpoint read, metadata), core/Weights_Storage/Weights_Storage.h:70-178 (worker attach),
// core/GPU_Weight_Buffer/replica_control_block.h:21-67 (barrier words, publication, abort).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

struct Region {
  void* base = nullptr;
  size_t bytes = 0;
  int fd = -1;
  bool owner = false;
};

constexpr int kMaxMembers = 8;
constexpr int kMaxTypes = 8;
constexpr int kMaxSlots = 64;
constexpr uint32_t kRcbMagic = 0x52434231;  // "RCB1"

struct ReplicaControl {
  uint32_t magic;
  uint32_t members;
  std::atomic<uint64_t> barrier_a[kMaxMembers][kMaxTypes];   // frames published by the member (as owner)
  std::atomic<uint64_t> barrier_b[kMaxMembers][kMaxTypes];   // frames the member has finished pulling
  std::atomic<uint64_t> slot_seq[kMaxMembers][kMaxSlots];    // publication sequence of each ring slot
  std::atomic<uint32_t> abort_flag[kMaxMembers];
};

template <class Pred>
bool wait_until(Pred p, int timeout_ms) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int spins = 0;
  while (!p()) {
    if (++spins > 200) {
      if (std::chrono::steady_clock::now() > deadline) return false;
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  return true;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ parameter store
void* bgc_pstore_create(unsigned long long bytes, int want_huge_pages, int* fd_out) {
  int fd = static_cast<int>(syscall(SYS_memfd_create, "bg_weights", 0));
  if (fd < 0) return nullptr;
  if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) { close(fd); return nullptr; }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) { close(fd); return nullptr; }
#ifdef MADV_HUGEPAGE
  if (want_huge_pages) madvise(p, bytes, MADV_HUGEPAGE);
#endif
  auto* r = new Region{p, static_cast<size_t>(bytes), fd, true};
  if (fd_out) *fd_out = fd;
  return r;
}

void* bgc_pstore_attach(int fd, int read_only) {
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size <= 0) return nullptr;
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | (read_only ? 0 : PROT_WRITE), MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) return nullptr;
  return new Region{p, static_cast<size_t>(st.st_size), fd, false};
}

void* bgc_pstore_base(void* r) { return static_cast<Region*>(r)->base; }
unsigned long long bgc_pstore_bytes(void* r) { return static_cast<Region*>(r)->bytes; }

// Read `n` files into the region at the given offsets with `threads` reader threads (each file in 16 MiB
// preads).  Returns 0, or -(index + 1) of the first file that failed.
int bgc_pstore_load_files(void* r, const char* const* paths, const unsigned long long* offsets,
                          const unsigned long long* sizes, int n, int threads) {
  Region* reg = static_cast<Region*>(r);
  std::atomic<int> next{0};
  std::atomic<int> failed{0};
  auto work = [&]() {
    for (;;) {
      const int i = next.fetch_add(1);
      if (i >= n) return;
      if (offsets[i] + sizes[i] > reg->bytes) { failed.store(-(i + 1)); continue; }
      int fd = open(paths[i], O_RDONLY);
      if (fd < 0) { failed.store(-(i + 1)); continue; }
      char* dst = static_cast<char*>(reg->base) + offsets[i];
      size_t done = 0;
      while (done < sizes[i]) {
        const size_t want = std::min<size_t>(sizes[i] - done, 16u << 20);
        const ssize_t got = pread(fd, dst + done, want, static_cast<off_t>(done));
        if (got <= 0) { failed.store(-(i + 1)); break; }
        done += static_cast<size_t>(got);
      }
      close(fd);
    }
  };
  std::vector<std::thread> pool;
  for (int t = 0; t < std::max(1, threads); ++t) pool.emplace_back(work);
  for (auto& t : pool) t.join();
  return failed.load();
}

void bgc_pstore_destroy(void* r) {
  Region* reg = static_cast<Region*>(r);
  if (reg->base) munmap(reg->base, reg->bytes);
  if (reg->owner && reg->fd >= 0) close(reg->fd);
  delete reg;
}

// ------------------------------------------------------------------ replica control block
unsigned long long bgc_rcb_bytes() { return sizeof(ReplicaControl); }

// `mem` is shared memory of at least bgc_rcb_bytes() (e.g. a parameter store region or any MAP_SHARED map)
int bgc_rcb_init(void* mem, int members) {
  if (members < 1 || members > kMaxMembers) return -1;
  auto* c = new (mem) ReplicaControl();
  c->members = static_cast<uint32_t>(members);
  for (int m = 0; m < kMaxMembers; ++m) {
    for (int t = 0; t < kMaxTypes; ++t) { c->barrier_a[m][t].store(0); c->barrier_b[m][t].store(0); }
    for (int s = 0; s < kMaxSlots; ++s) c->slot_seq[m][s].store(0);
    c->abort_flag[m].store(0);
  }
  std::atomic_thread_fence(std::memory_order_release);
  c->magic = kRcbMagic;
  return 0;
}

static ReplicaControl* rcb(void* mem) {
  auto* c = static_cast<ReplicaControl*>(mem);
  return c->magic == kRcbMagic ? c : nullptr;
}

// owner: slot `slot` of my ring now holds frame `frame` of module type `type`
int bgc_rcb_publish(void* mem, int member, int type, int slot, unsigned long long frame) {
  ReplicaControl* c = rcb(mem);
  if (!c || member < 0 || member >= (int)c->members || type < 0 || type >= kMaxTypes || slot < 0 || slot >= kMaxSlots) return -1;
  c->slot_seq[member][slot].store(frame, std::memory_order_release);
  c->barrier_a[member][type].store(frame, std::memory_order_release);
  return 0;
}

// reader: wait until `owner` has published at least `frame` of `type` (barrier A).  0 ok, 1 timeout, 2 aborted
int bgc_rcb_wait_published(void* mem, int owner, int type, unsigned long long frame, int timeout_ms) {
  ReplicaControl* c = rcb(mem);
  if (!c) return -1;
  bool aborted = false;
  const bool ok = wait_until([&] {
    if (c->abort_flag[owner].load(std::memory_order_acquire)) { aborted = true; return true; }
    return c->barrier_a[owner][type].load(std::memory_order_acquire) >= frame;
  }, timeout_ms);
  return aborted ? 2 : (ok ? 0 : 1);
}

// reader: I have pulled frame `frame` of `type`
int bgc_rcb_ack_pulled(void* mem, int member, int type, unsigned long long frame) {
  ReplicaControl* c = rcb(mem);
  if (!c) return -1;
  c->barrier_b[member][type].store(frame, std::memory_order_release);
  return 0;
}

// owner: wait until every other member has pulled at least `frame` of `type` (barrier B) before slot reuse
int bgc_rcb_wait_all_pulled(void* mem, int owner, int type, unsigned long long frame, int timeout_ms) {
  ReplicaControl* c = rcb(mem);
  if (!c) return -1;
  bool aborted = false;
  const bool ok = wait_until([&] {
    for (uint32_t m = 0; m < c->members; ++m)
      if ((int)m != owner && c->abort_flag[m].load(std::memory_order_acquire)) { aborted = true; return true; }
    for (uint32_t m = 0; m < c->members; ++m)
      if ((int)m != owner && c->barrier_b[m][type].load(std::memory_order_acquire) < frame) return false;
    return true;
  }, timeout_ms);
  return aborted ? 2 : (ok ? 0 : 1);
}

unsigned long long bgc_rcb_slot_frame(void* mem, int member, int slot) {
  ReplicaControl* c = rcb(mem);
  return c ? c->slot_seq[member][slot].load(std::memory_order_acquire) : 0;
}

int bgc_rcb_abort(void* mem, int member) {
  ReplicaControl* c = rcb(mem);
  if (!c) return -1;
  c->abort_flag[member].store(1, std::memory_order_release);
  return 0;
}

}  // extern "C"

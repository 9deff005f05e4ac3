// Node weight daemon of a distributed host weight store.
//
// Each node keeps a share of the checkpoint's modules in host memory (its "local store").  Workers of a node ask
// their daemon for modules over a unix socket: a local module is answered with its place in the local store, a
// remote one with a slot of the node's staging region that holds a copy fetched from the owning node.  A prefetch
// thread walks the cyclic module schedule ahead of the workers and fills free staging slots, so an acquire that
// follows the schedule finds its module ready.
//
// Worker protocol (fixed-size little-endian records, one reply per request):
//   hello(worker, epoch)   admitted only for the cohort epoch the daemon serves and while no swap is open
//   acquire(key)           local: status 0, slot -1, offset into the local store; remote and ready: status 0 with
//                          a leased slot; not ready within one bounded wait: status kRetry (nothing acquired)
//   release(key)           drops one lease of the connection on the module's slot
// A connection that closes gives its leases back.
//
// Node transport: a TCP listener serves "get(key)" to the other nodes' daemons out of the local store (the place a
// one-sided RMA transport would take; the byte stream is length-prefixed and checked).  A failed transfer latches
// `transport_failed`: acquires of remote modules then fail and only a restart clears it.
//
// Cohort swap (the server replaces its workers while the daemon stays up): begin_swap() stops admitting hellos and
// fails pending and new acquires; finish_swap() closes every connection, frees all leases and slots, rewinds the
// schedule and admits the next epoch.
//
// Reference parity: core/Weights_Storage/distributed_weight_daemon.{h,cpp} (daemon, prefetch ring, cohort swap,
// status), distributed_weights_protocol.h (hello / acquire / release, retry status), latency_histogram.h.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace bgcore {

constexpr uint64_t kDaemonMagic = 0x4247574431303031ull;   // "BGWD1001"
constexpr int32_t kStatusRetry = 1;
constexpr size_t kKeyBytes = 64;

enum DaemonOp : uint32_t { kOpHello = 1, kOpAcquire = 2, kOpRelease = 3 };

struct DaemonRequest {
  uint64_t magic = kDaemonMagic;
  uint32_t op = 0;
  uint32_t worker = 0;
  uint64_t epoch = 0;
  char key[kKeyBytes] = {};
};

struct DaemonResponse {
  uint64_t magic = kDaemonMagic;
  int32_t status = 0;         // 0 ok, kStatusRetry, negative = error that ends the connection
  int32_t slot = -1;          // staging slot, or -1 for a local module
  uint64_t epoch = 0;
  uint64_t offset = 0;        // byte offset in the local store (slot < 0) or in the staging region
  uint64_t bytes = 0;         // module bytes
  char error[96] = {};
};

// Log-spaced latency histogram (16 buckets per octave from about a microsecond to minutes); percentile() returns
// the upper edge of the bucket that holds the nearest rank.
class LatencyHistogram {
 public:
  void record(double ms);
  double percentile(double pct) const;
  double max() const { return max_; }
  uint64_t count() const { return count_; }
  double mean() const { return count_ ? sum_ / (double)count_ : 0.0; }

 private:
  static constexpr int kSub = 16, kMinOct = -10, kMaxOct = 19, kBuckets = (kMaxOct - kMinOct) * kSub + 2;
  static int bucket_of(double ms);
  uint64_t counts_[kBuckets] = {};
  uint64_t count_ = 0;
  double sum_ = 0, max_ = 0;
};

struct DaemonConfig {
  int node = 0;
  std::string socket_path;                         // unix socket of the worker protocol
  int listen_port = 0;                             // TCP port of the node transport (0 = none: single node)
  std::map<int, std::string> peers;                // node -> "host:port"
  int staging_slots = 4;
  uint64_t slot_bytes = 0;
  int prefetch_depth = 2;                          // remote modules kept ready ahead of the cursor
  int acquire_wait_ms = 50;                        // one bounded wait of an acquire before kRetry
};

struct ModuleInfo {
  int owner = 0;
  uint64_t offset = 0;      // in the owner's local store
  uint64_t bytes = 0;
};

class WeightDaemon {
 public:
  explicit WeightDaemon(const DaemonConfig& cfg);
  ~WeightDaemon();
  // Before start(): the local store (memory owned by the caller, alive until stop()) and the module directory of the
  // whole model (every node registers the same directory), then the cyclic schedule of module keys.
  void set_local_store(const void* base, uint64_t bytes);
  bool add_module(const std::string& key, int owner, uint64_t offset, uint64_t bytes);
  void set_schedule(const std::vector<std::string>& keys);
  bool start();                                     // false: a socket could not be opened
  void stop();
  int staging_fd() const { return staging_fd_; }
  uint64_t staging_bytes() const { return (uint64_t)cfg_.staging_slots * cfg_.slot_bytes; }
  uint64_t epoch();
  uint64_t begin_swap();
  std::string finish_swap();                        // JSON report of what was released
  std::string status();                             // JSON

 private:
  enum SlotState { kFree = 0, kFetching = 1, kReady = 2 };
  struct Slot {
    SlotState state = kFree;
    std::string key;
    int leases = 0;
    uint64_t stamp = 0;     // schedule position it was fetched for
  };
  struct Conn {
    int fd = -1;
    std::thread th;
    std::map<int, int> leases;     // slot -> count
    bool admitted = false;
    std::atomic<bool> done{false};
  };

  void accept_loop();
  void serve_worker(Conn* c);
  void transport_loop();
  void serve_peer(int fd);
  void prefetch_loop();
  bool fetch_into(int slot, const std::string& key, const ModuleInfo& mi);
  int find_slot_locked(const std::string& key) const;
  int take_free_slot_locked(uint64_t cursor);
  void advance_cursor_locked(const std::string& key);
  DaemonResponse do_acquire(Conn* c, const std::string& key);
  void release_conn_leases_locked(Conn* c);
  void close_conns(bool join);

  DaemonConfig cfg_;
  const uint8_t* store_ = nullptr;
  uint64_t store_bytes_ = 0;
  std::map<std::string, ModuleInfo> modules_;
  std::vector<std::string> schedule_;
  int staging_fd_ = -1;
  uint8_t* staging_ = nullptr;

  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<Slot> slots_;
  uint64_t cursor_ = 0;                 // schedule position of the next expected acquire
  // remote modules a worker is waiting for -> time of its last request.  An entry lives until the module is leased
  // (or the worker stops asking): its slot is not a prefetch victim in between.
  std::map<std::string, std::chrono::steady_clock::time_point> demand_;
  std::map<int, int> peer_fds_;         // owner node -> connection (prefetch thread only)
  uint64_t epoch_ = 1;
  bool swap_open_ = false;
  int swap_released_ = 0;               // leases given back by connections that ended while the swap was open
  std::string cohort_fault_;
  std::atomic<bool> transport_failed_{false};
  std::atomic<bool> stop_{false};
  bool started_ = false;

  int listen_unix_ = -1, listen_tcp_ = -1;
  std::thread accept_th_, transport_th_, prefetch_th_;
  std::mutex conn_mu_;
  std::vector<Conn*> conns_;
  std::vector<std::thread> peer_threads_;

  std::mutex stats_mu_;
  uint64_t n_acquire_ = 0, n_local_ = 0, n_hit_ = 0, n_retry_ = 0, n_fetch_ = 0, n_demand_fetch_ = 0;
  uint64_t bytes_fetched_ = 0, bytes_served_ = 0, n_hello_refused_ = 0;
  LatencyHistogram fetch_ms_, acquire_ms_;
};

// Worker side of the protocol: one blocking connection.
class DaemonClient {
 public:
  ~DaemonClient();
  bool connect_to(const std::string& socket_path);
  // -> 0 admitted, negative refused (error text in last_error()).
  int hello(uint32_t worker, uint64_t epoch);
  // Re-sends while the daemon answers kRetry, up to timeout_ms.  -> 0 and fills the outputs, kStatusRetry on
  // timeout, negative on error.
  int acquire(const std::string& key, int timeout_ms, int* slot, uint64_t* offset, uint64_t* bytes);
  int release(const std::string& key);
  void close_conn();
  const std::string& last_error() const { return err_; }

 private:
  bool roundtrip(const DaemonRequest& rq, DaemonResponse* rs);
  int fd_ = -1;
  uint32_t worker_ = 0;
  uint64_t epoch_ = 0;
  std::string err_;
};

}  // namespace bgcore

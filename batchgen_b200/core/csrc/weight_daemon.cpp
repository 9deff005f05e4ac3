#include "weight_daemon.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <sstream>

namespace bgcore {

namespace {

using Clock = std::chrono::steady_clock;

double ms_since(Clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

// Reads / writes exactly n bytes, waking every 200 ms to look at `stop`.  false: closed, error or stopped.
bool read_full(int fd, void* buf, size_t n, const std::atomic<bool>* stop) {
  auto* p = static_cast<uint8_t*>(buf);
  while (n > 0) {
    pollfd pf{fd, POLLIN, 0};
    const int rc = ::poll(&pf, 1, 200);
    if (stop != nullptr && stop->load()) return false;
    if (rc < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    if (rc == 0) continue;
    const ssize_t got = ::read(fd, p, n);
    if (got == 0) return false;
    if (got < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return false;
    }
    p += got;
    n -= (size_t)got;
  }
  return true;
}

bool write_full(int fd, const void* buf, size_t n) {
  auto* p = static_cast<const uint8_t*>(buf);
  while (n > 0) {
    const ssize_t put = ::send(fd, p, n, MSG_NOSIGNAL);
    if (put < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += put;
    n -= (size_t)put;
  }
  return true;
}

struct PeerRequest {
  uint64_t magic = kDaemonMagic;
  char key[kKeyBytes] = {};
};

struct PeerReply {
  uint64_t magic = kDaemonMagic;
  int64_t status = 0;      // 0 ok, -1 unknown / not local
  uint64_t bytes = 0;
};

void set_key(char* dst, const std::string& key) {
  std::memset(dst, 0, kKeyBytes);
  std::memcpy(dst, key.data(), std::min(key.size(), kKeyBytes - 1));
}

std::string get_key(const char* src) { return std::string(src, strnlen(src, kKeyBytes)); }

void set_error(DaemonResponse* rs, int32_t status, const std::string& msg) {
  rs->status = status;
  std::memset(rs->error, 0, sizeof(rs->error));
  std::memcpy(rs->error, msg.data(), std::min(msg.size(), sizeof(rs->error) - 1));
}

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') o.push_back('\\');
    o.push_back(c == '\n' ? ' ' : c);
  }
  return o;
}

}  // namespace

// ---------------------------------------------------------------- LatencyHistogram
int LatencyHistogram::bucket_of(double ms) {
  if (!(ms > std::ldexp(1.0, kMinOct))) return 0;
  if (ms > std::ldexp(1.0, kMaxOct)) return kBuckets - 1;
  const int k = (int)std::ceil((std::log2(ms) - kMinOct) * kSub);
  return std::min(std::max(k, 1), kBuckets - 2);
}

void LatencyHistogram::record(double ms) {
  counts_[bucket_of(ms)]++;
  count_++;
  sum_ += ms;
  max_ = std::max(max_, ms);
}

double LatencyHistogram::percentile(double pct) const {
  if (count_ == 0) return 0.0;
  uint64_t rank = (uint64_t)std::ceil(pct * (double)count_ / 100.0);
  rank = std::min(std::max<uint64_t>(rank, 1), count_);
  uint64_t seen = 0;
  for (int b = 0; b < kBuckets; ++b) {
    seen += counts_[b];
    if (seen >= rank) {
      if (b == 0) return std::ldexp(1.0, kMinOct);
      if (b == kBuckets - 1) return std::ldexp(1.0, kMaxOct);
      return std::exp2(kMinOct + (double)b / kSub);
    }
  }
  return max_;
}

// ---------------------------------------------------------------- WeightDaemon
WeightDaemon::WeightDaemon(const DaemonConfig& cfg) : cfg_(cfg), slots_(std::max(cfg.staging_slots, 0)) {}

WeightDaemon::~WeightDaemon() { stop(); }

void WeightDaemon::set_local_store(const void* base, uint64_t bytes) {
  store_ = static_cast<const uint8_t*>(base);
  store_bytes_ = bytes;
}

bool WeightDaemon::add_module(const std::string& key, int owner, uint64_t offset, uint64_t bytes) {
  if (key.empty() || key.size() >= kKeyBytes) return false;
  if (owner == cfg_.node && offset + bytes > store_bytes_) return false;
  if (owner != cfg_.node && bytes > cfg_.slot_bytes) return false;     // must fit a staging slot
  modules_[key] = ModuleInfo{owner, offset, bytes};
  return true;
}

void WeightDaemon::set_schedule(const std::vector<std::string>& keys) { schedule_ = keys; }

bool WeightDaemon::start() {
  if (started_) return true;
  if (cfg_.staging_slots > 0 && cfg_.slot_bytes > 0) {
    staging_fd_ = (int)::syscall(SYS_memfd_create, "bg_weight_staging", 0u);
    if (staging_fd_ < 0 || ::ftruncate(staging_fd_, (off_t)staging_bytes()) != 0) return false;
    void* p = ::mmap(nullptr, staging_bytes(), PROT_READ | PROT_WRITE, MAP_SHARED, staging_fd_, 0);
    if (p == MAP_FAILED) return false;
    staging_ = static_cast<uint8_t*>(p);
  }
  listen_unix_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un ua{};
  ua.sun_family = AF_UNIX;
  if (listen_unix_ < 0 || cfg_.socket_path.size() >= sizeof(ua.sun_path)) return false;
  std::strcpy(ua.sun_path, cfg_.socket_path.c_str());
  ::unlink(cfg_.socket_path.c_str());
  if (::bind(listen_unix_, reinterpret_cast<sockaddr*>(&ua), sizeof(ua)) != 0 || ::listen(listen_unix_, 64) != 0) return false;
  if (cfg_.listen_port > 0) {
    listen_tcp_ = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    ::setsockopt(listen_tcp_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in ia{};
    ia.sin_family = AF_INET;
    ia.sin_addr.s_addr = htonl(INADDR_ANY);
    ia.sin_port = htons((uint16_t)cfg_.listen_port);
    if (listen_tcp_ < 0 || ::bind(listen_tcp_, reinterpret_cast<sockaddr*>(&ia), sizeof(ia)) != 0 ||
        ::listen(listen_tcp_, 64) != 0)
      return false;
    transport_th_ = std::thread([this] { transport_loop(); });
  }
  stop_ = false;
  accept_th_ = std::thread([this] { accept_loop(); });
  prefetch_th_ = std::thread([this] { prefetch_loop(); });
  started_ = true;
  return true;
}

void WeightDaemon::stop() {
  if (!started_) {                       // start() gave up half way: give back what it had opened
    if (listen_unix_ >= 0) ::close(listen_unix_);
    if (listen_tcp_ >= 0) ::close(listen_tcp_);
    listen_unix_ = listen_tcp_ = -1;
    if (staging_ != nullptr) ::munmap(staging_, staging_bytes());
    if (staging_fd_ >= 0) ::close(staging_fd_);
    staging_ = nullptr;
    staging_fd_ = -1;
    return;
  }
  stop_ = true;
  cv_.notify_all();
  if (accept_th_.joinable()) accept_th_.join();
  if (transport_th_.joinable()) transport_th_.join();
  if (prefetch_th_.joinable()) prefetch_th_.join();
  for (auto& t : peer_threads_)
    if (t.joinable()) t.join();
  peer_threads_.clear();
  close_conns(true);
  if (listen_unix_ >= 0) ::close(listen_unix_);
  if (listen_tcp_ >= 0) ::close(listen_tcp_);
  listen_unix_ = listen_tcp_ = -1;
  ::unlink(cfg_.socket_path.c_str());
  if (staging_ != nullptr) ::munmap(staging_, staging_bytes());
  if (staging_fd_ >= 0) ::close(staging_fd_);
  staging_ = nullptr;
  staging_fd_ = -1;
  started_ = false;
}

void WeightDaemon::close_conns(bool join) {
  std::vector<Conn*> conns;
  {
    std::lock_guard<std::mutex> g(conn_mu_);
    conns.swap(conns_);
  }
  for (Conn* c : conns) {
    c->done = true;
    if (c->fd >= 0) ::shutdown(c->fd, SHUT_RDWR);
  }
  for (Conn* c : conns) {
    if (join && c->th.joinable()) c->th.join();
    if (c->fd >= 0) ::close(c->fd);
    {
      std::lock_guard<std::mutex> g(mu_);
      release_conn_leases_locked(c);
    }
    delete c;
  }
}

void WeightDaemon::accept_loop() {
  while (!stop_) {
    pollfd pf{listen_unix_, POLLIN, 0};
    const int rc = ::poll(&pf, 1, 200);
    {   // reap connections whose worker went away
      std::lock_guard<std::mutex> g(conn_mu_);
      for (size_t i = 0; i < conns_.size();) {
        Conn* c = conns_[i];
        if (c->done && c->th.joinable()) {
          c->th.join();
          ::close(c->fd);
          delete c;
          conns_.erase(conns_.begin() + i);
        } else {
          ++i;
        }
      }
    }
    if (rc <= 0) continue;
    const int fd = ::accept(listen_unix_, nullptr, nullptr);
    if (fd < 0) continue;
    auto* c = new Conn();
    c->fd = fd;
    {
      std::lock_guard<std::mutex> g(conn_mu_);        // the thread handle is written before anyone can look at it
      c->th = std::thread([this, c] { serve_worker(c); });
      conns_.push_back(c);
    }
  }
}

void WeightDaemon::release_conn_leases_locked(Conn* c) {
  for (auto& kv : c->leases) {
    if (kv.first >= 0 && kv.first < (int)slots_.size()) slots_[kv.first].leases = std::max(0, slots_[kv.first].leases - kv.second);
    if (swap_open_) swap_released_ += kv.second;
  }
  c->leases.clear();
  cv_.notify_all();
}

int WeightDaemon::find_slot_locked(const std::string& key) const {
  for (size_t i = 0; i < slots_.size(); ++i)
    if (slots_[i].state != kFree && slots_[i].key == key) return (int)i;
  return -1;
}

void WeightDaemon::advance_cursor_locked(const std::string& key) {
  const size_t n = schedule_.size();
  if (n == 0) return;
  for (size_t j = 0; j < n; ++j) {
    if (schedule_[(cursor_ + j) % n] == key) {
      cursor_ += j + 1;
      cv_.notify_all();
      return;
    }
  }
}

DaemonResponse WeightDaemon::do_acquire(Conn* c, const std::string& key) {
  DaemonResponse rs;
  const auto t0 = Clock::now();
  std::unique_lock<std::mutex> lk(mu_);
  rs.epoch = epoch_;
  if (swap_open_) {
    set_error(&rs, -2, "cohort swap in progress");
    return rs;
  }
  auto it = modules_.find(key);
  if (it == modules_.end()) {
    set_error(&rs, -3, "unknown module " + key);
    return rs;
  }
  const ModuleInfo mi = it->second;
  {
    std::lock_guard<std::mutex> g(stats_mu_);
    n_acquire_++;
  }
  rs.bytes = mi.bytes;
  if (mi.owner == cfg_.node) {
    rs.slot = -1;
    rs.offset = mi.offset;
    advance_cursor_locked(key);
    std::lock_guard<std::mutex> g(stats_mu_);
    n_local_++;
    return rs;
  }
  if (transport_failed_) {
    set_error(&rs, -4, "node transport failed; the daemon needs a restart");
    return rs;
  }
  int slot = find_slot_locked(key);
  const bool ready_now = slot >= 0 && slots_[slot].state == kReady;
  if (!ready_now) {
    demand_[key] = Clock::now();
    cv_.notify_all();
    const auto deadline = Clock::now() + std::chrono::milliseconds(cfg_.acquire_wait_ms);
    cv_.wait_until(lk, deadline, [&] {
      if (stop_ || swap_open_ || transport_failed_) return true;
      const int s = find_slot_locked(key);
      return s >= 0 && slots_[s].state == kReady;
    });
    if (swap_open_ || stop_) {
      set_error(&rs, -2, "cohort swap in progress");
      return rs;
    }
    if (transport_failed_) {
      set_error(&rs, -4, "node transport failed; the daemon needs a restart");
      return rs;
    }
    slot = find_slot_locked(key);
    if (slot < 0 || slots_[slot].state != kReady) {
      rs.status = kStatusRetry;
      std::lock_guard<std::mutex> g(stats_mu_);
      n_retry_++;
      return rs;
    }
  }
  slots_[slot].leases++;
  c->leases[slot]++;
  demand_.erase(key);
  advance_cursor_locked(key);          // the schedule moves on successful acquires only (a retry is the same step)
  rs.slot = slot;
  rs.offset = (uint64_t)slot * cfg_.slot_bytes;
  std::lock_guard<std::mutex> g(stats_mu_);
  if (ready_now) n_hit_++;
  acquire_ms_.record(ms_since(t0));
  return rs;
}

void WeightDaemon::serve_worker(Conn* c) {
  while (!stop_ && !c->done) {
    DaemonRequest rq;
    if (!read_full(c->fd, &rq, sizeof(rq), &stop_)) break;
    DaemonResponse rs;
    if (rq.magic != kDaemonMagic) {
      set_error(&rs, -9, "bad magic");
      write_full(c->fd, &rs, sizeof(rs));
      break;
    }
    const std::string key = get_key(rq.key);
    if (rq.op == kOpHello) {
      std::lock_guard<std::mutex> g(mu_);
      rs.epoch = epoch_;
      if (swap_open_ || rq.epoch != epoch_) {
        set_error(&rs, -1, swap_open_ ? "cohort swap in progress" : "wrong cohort epoch");
        std::lock_guard<std::mutex> s(stats_mu_);
        n_hello_refused_++;
      } else {
        c->admitted = true;
      }
    } else if (!c->admitted) {
      set_error(&rs, -5, "hello first");
    } else if (rq.op == kOpAcquire) {
      rs = do_acquire(c, key);
    } else if (rq.op == kOpRelease) {
      std::lock_guard<std::mutex> g(mu_);
      rs.epoch = epoch_;
      const int slot = find_slot_locked(key);
      auto it = slot >= 0 ? c->leases.find(slot) : c->leases.end();
      if (it != c->leases.end() && it->second > 0) {
        if (--it->second == 0) c->leases.erase(it);
        slots_[slot].leases = std::max(0, slots_[slot].leases - 1);
        cv_.notify_all();
      } else if (modules_.count(key) == 0 || modules_[key].owner != cfg_.node) {
        set_error(&rs, -6, "no lease on " + key);
      }
    } else {
      set_error(&rs, -7, "unknown operation");
    }
    if (!write_full(c->fd, &rs, sizeof(rs))) break;
    if (rs.status < 0 && rs.status != -6) break;         // errors end the connection (a stray release does not)
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    release_conn_leases_locked(c);
  }
  ::shutdown(c->fd, SHUT_RDWR);
  c->done = true;
}

int WeightDaemon::take_free_slot_locked(uint64_t cursor) {
  for (size_t i = 0; i < slots_.size(); ++i)
    if (slots_[i].state == kFree) return (int)i;
  // evict the unleased ready slot whose module is used farthest in the future
  const size_t n = schedule_.size();
  int best = -1;
  size_t best_dist = 0;
  for (size_t i = 0; i < slots_.size(); ++i) {
    if (slots_[i].state != kReady || slots_[i].leases > 0) continue;
    size_t dist = n + 1;
    for (size_t j = 0; j < n; ++j)
      if (schedule_[(cursor + j) % n] == slots_[i].key) {
        dist = j;
        break;
      }
    if (best < 0 || dist > best_dist) {
      best = (int)i;
      best_dist = dist;
    }
  }
  return best;
}

void WeightDaemon::prefetch_loop() {
  while (!stop_) {
    std::string key;
    int slot = -1;
    ModuleInfo mi;
    bool demand = false;
    {
      std::unique_lock<std::mutex> lk(mu_);
      if (!swap_open_ && !transport_failed_) {
        // what should be resident: demanded modules first, then the next remote modules of the schedule
        std::vector<std::string> want;
        for (auto it = demand_.begin(); it != demand_.end();) {
          if (ms_since(it->second) > 2000.0) {
            it = demand_.erase(it);                 // the worker stopped asking
          } else {
            want.push_back(it->first);
            ++it;
          }
        }
        const size_t n = schedule_.size();
        int ahead = 0;
        for (size_t j = 0; j < n && ahead < cfg_.prefetch_depth; ++j) {
          const std::string& k = schedule_[(cursor_ + j) % n];
          auto it = modules_.find(k);
          if (it == modules_.end() || it->second.owner == cfg_.node) continue;
          if (std::find(want.begin(), want.end(), k) == want.end()) want.push_back(k);
          ++ahead;
        }
        for (const auto& k : want) {
          if (find_slot_locked(k) >= 0) continue;
          // a slot that holds a wanted module is not a victim
          int s = -1;
          for (size_t i = 0; i < slots_.size() && s < 0; ++i)
            if (slots_[i].state == kFree) s = (int)i;
          if (s < 0) {
            const int cand = take_free_slot_locked(cursor_);
            if (cand >= 0 && std::find(want.begin(), want.end(), slots_[cand].key) == want.end()) s = cand;
          }
          if (s < 0) continue;
          key = k;
          slot = s;
          mi = modules_[k];
          demand = demand_.count(k) > 0;
          slots_[s].state = kFetching;
          slots_[s].key = k;
          slots_[s].leases = 0;
          slots_[s].stamp = cursor_;
          break;
        }
      }
      if (slot < 0) {
        cv_.wait_for(lk, std::chrono::milliseconds(50));
        continue;
      }
    }
    const auto t0 = Clock::now();
    const bool ok = fetch_into(slot, key, mi);
    {
      std::lock_guard<std::mutex> g(mu_);
      if (ok) {
        slots_[slot].state = kReady;
      } else {
        slots_[slot] = Slot();
        if (!stop_) {
          transport_failed_ = true;
          cohort_fault_ = "fetch of " + key + " from node " + std::to_string(mi.owner) + " failed";
        }
      }
      cv_.notify_all();
    }
    if (ok) {
      std::lock_guard<std::mutex> g(stats_mu_);
      n_fetch_++;
      if (demand) n_demand_fetch_++;
      bytes_fetched_ += mi.bytes;
      fetch_ms_.record(ms_since(t0));
    }
  }
  for (auto& kv : peer_fds_) ::close(kv.second);
  peer_fds_.clear();
}

bool WeightDaemon::fetch_into(int slot, const std::string& key, const ModuleInfo& mi) {
  if (staging_ == nullptr || mi.bytes > cfg_.slot_bytes) return false;
  auto pit = cfg_.peers.find(mi.owner);
  if (pit == cfg_.peers.end()) return false;
  for (int attempt = 0; attempt < 2; ++attempt) {
    int fd = -1;
    auto fit = peer_fds_.find(mi.owner);
    if (fit != peer_fds_.end()) {
      fd = fit->second;
    } else {
      const std::string& addr = pit->second;
      const size_t colon = addr.rfind(':');
      if (colon == std::string::npos) return false;
      addrinfo hints{}, *res = nullptr;
      hints.ai_family = AF_INET;
      hints.ai_socktype = SOCK_STREAM;
      if (::getaddrinfo(addr.substr(0, colon).c_str(), addr.substr(colon + 1).c_str(), &hints, &res) != 0 || res == nullptr) return false;
      fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      // the owner may still be starting: retry the connect for a few seconds
      bool connected = false;
      for (int i = 0; i < 50 && fd >= 0 && !stop_; ++i) {
        if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
          connected = true;
          break;
        }
        ::usleep(100 * 1000);
      }
      ::freeaddrinfo(res);
      if (!connected) {
        if (fd >= 0) ::close(fd);
        return false;
      }
      int one = 1;
      ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      peer_fds_[mi.owner] = fd;
    }
    PeerRequest rq;
    set_key(rq.key, key);
    PeerReply rp;
    if (write_full(fd, &rq, sizeof(rq)) && read_full(fd, &rp, sizeof(rp), &stop_) && rp.magic == kDaemonMagic &&
        rp.status == 0 && rp.bytes == mi.bytes &&
        read_full(fd, staging_ + (uint64_t)slot * cfg_.slot_bytes, mi.bytes, &stop_))
      return true;
    ::close(fd);                       // a stale connection: reconnect once
    peer_fds_.erase(mi.owner);
  }
  return false;
}

void WeightDaemon::transport_loop() {
  while (!stop_) {
    pollfd pf{listen_tcp_, POLLIN, 0};
    if (::poll(&pf, 1, 200) <= 0) continue;
    const int fd = ::accept(listen_tcp_, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    peer_threads_.emplace_back([this, fd] { serve_peer(fd); });
  }
}

void WeightDaemon::serve_peer(int fd) {
  while (!stop_) {
    PeerRequest rq;
    if (!read_full(fd, &rq, sizeof(rq), &stop_) || rq.magic != kDaemonMagic) break;
    PeerReply rp;
    auto it = modules_.find(get_key(rq.key));
    if (it == modules_.end() || it->second.owner != cfg_.node || store_ == nullptr) {
      rp.status = -1;
      write_full(fd, &rp, sizeof(rp));
      continue;
    }
    rp.bytes = it->second.bytes;
    if (!write_full(fd, &rp, sizeof(rp)) || !write_full(fd, store_ + it->second.offset, it->second.bytes)) break;
    std::lock_guard<std::mutex> g(stats_mu_);
    bytes_served_ += it->second.bytes;
  }
  ::close(fd);
}

uint64_t WeightDaemon::epoch() {
  std::lock_guard<std::mutex> g(mu_);
  return epoch_;
}

uint64_t WeightDaemon::begin_swap() {
  std::lock_guard<std::mutex> g(mu_);
  if (!swap_open_) swap_released_ = 0;
  swap_open_ = true;
  cv_.notify_all();
  return epoch_;
}

std::string WeightDaemon::finish_swap() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!swap_open_) return "{\"ok\": false, \"error\": \"no swap is open\"}";
  }
  size_t conns = 0;
  {
    std::lock_guard<std::mutex> g(conn_mu_);
    conns = conns_.size();
  }
  close_conns(true);
  std::unique_lock<std::mutex> lk(mu_);
  // a fetch in flight finishes (bounded) before its slot is reused
  cv_.wait_for(lk, std::chrono::seconds(10), [&] {
    for (const auto& s : slots_)
      if (s.state == kFetching) return false;
    return true;
  });
  int leases = swap_released_, ready = 0;
  for (auto& s : slots_) {
    leases += s.leases;
    ready += s.state == kReady;
    s = Slot();
  }
  const uint64_t from = cursor_;
  cursor_ = 0;
  demand_.clear();
  const bool failed = transport_failed_;
  if (!failed) cohort_fault_.clear();
  const uint64_t old_epoch = epoch_;
  if (!failed) {
    epoch_++;
    swap_open_ = false;
  }
  cv_.notify_all();
  std::ostringstream o;
  o << "{\"ok\": " << (failed ? "false" : "true") << ", \"old_epoch\": " << old_epoch << ", \"epoch\": " << epoch_
    << ", \"connections_closed\": " << conns << ", \"leases_released\": " << leases << ", \"slots_freed\": " << ready
    << ", \"prefetch_cursor_rewound_from\": " << from << ", \"transport_failed\": " << (failed ? "true" : "false") << "}";
  return o.str();
}

std::string WeightDaemon::status() {
  std::ostringstream o;
  {
    std::lock_guard<std::mutex> g(mu_);
    int free_s = 0, fetching = 0, ready = 0, leased = 0;
    for (const auto& s : slots_) {
      free_s += s.state == kFree;
      fetching += s.state == kFetching;
      ready += s.state == kReady;
      leased += s.leases > 0;
    }
    o << "{\"node\": " << cfg_.node << ", \"epoch\": " << epoch_ << ", \"swap_open\": " << (swap_open_ ? "true" : "false")
      << ", \"transport_failed\": " << (transport_failed_ ? "true" : "false") << ", \"cohort_fault\": \""
      << json_escape(cohort_fault_) << "\", \"cursor\": " << cursor_ << ", \"slots\": {\"free\": " << free_s
      << ", \"fetching\": " << fetching << ", \"ready\": " << ready << ", \"leased\": " << leased << "}";
  }
  std::lock_guard<std::mutex> g(stats_mu_);
  o << ", \"acquires\": " << n_acquire_ << ", \"local\": " << n_local_ << ", \"ready_hits\": " << n_hit_
    << ", \"retries\": " << n_retry_ << ", \"fetches\": " << n_fetch_ << ", \"demand_fetches\": " << n_demand_fetch_
    << ", \"bytes_fetched\": " << bytes_fetched_ << ", \"bytes_served\": " << bytes_served_
    << ", \"hellos_refused\": " << n_hello_refused_ << ", \"fetch_ms\": {\"count\": " << fetch_ms_.count()
    << ", \"mean\": " << fetch_ms_.mean() << ", \"p50\": " << fetch_ms_.percentile(50) << ", \"p99\": "
    << fetch_ms_.percentile(99) << ", \"max\": " << fetch_ms_.max() << "}, \"acquire_ms\": {\"count\": "
    << acquire_ms_.count() << ", \"p50\": " << acquire_ms_.percentile(50) << ", \"p99\": " << acquire_ms_.percentile(99)
    << ", \"max\": " << acquire_ms_.max() << "}}";
  return o.str();
}

// ---------------------------------------------------------------- DaemonClient
DaemonClient::~DaemonClient() { close_conn(); }

void DaemonClient::close_conn() {
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
}

bool DaemonClient::connect_to(const std::string& socket_path) {
  close_conn();
  fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un ua{};
  ua.sun_family = AF_UNIX;
  if (fd_ < 0 || socket_path.size() >= sizeof(ua.sun_path)) return false;
  std::strcpy(ua.sun_path, socket_path.c_str());
  if (::connect(fd_, reinterpret_cast<sockaddr*>(&ua), sizeof(ua)) != 0) {
    close_conn();
    return false;
  }
  timeval tv{30, 0};
  ::setsockopt(fd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  return true;
}

bool DaemonClient::roundtrip(const DaemonRequest& rq, DaemonResponse* rs) {
  if (fd_ < 0) {
    err_ = "not connected";
    return false;
  }
  if (!write_full(fd_, &rq, sizeof(rq)) || !read_full(fd_, rs, sizeof(*rs), nullptr) || rs->magic != kDaemonMagic) {
    err_ = "connection to the weight daemon lost";
    close_conn();
    return false;
  }
  if (rs->status < 0) err_ = std::string(rs->error, strnlen(rs->error, sizeof(rs->error)));
  return true;
}

int DaemonClient::hello(uint32_t worker, uint64_t epoch) {
  DaemonRequest rq;
  rq.op = kOpHello;
  rq.worker = worker_ = worker;
  rq.epoch = epoch_ = epoch;
  DaemonResponse rs;
  if (!roundtrip(rq, &rs)) return -100;
  return rs.status;
}

int DaemonClient::acquire(const std::string& key, int timeout_ms, int* slot, uint64_t* offset, uint64_t* bytes) {
  const auto t0 = Clock::now();
  for (;;) {
    DaemonRequest rq;
    rq.op = kOpAcquire;
    rq.worker = worker_;
    rq.epoch = epoch_;
    set_key(rq.key, key);
    DaemonResponse rs;
    if (!roundtrip(rq, &rs)) return -100;
    if (rs.status == kStatusRetry) {
      if (ms_since(t0) > timeout_ms) return kStatusRetry;
      continue;
    }
    if (rs.status == 0) {
      *slot = rs.slot;
      *offset = rs.offset;
      *bytes = rs.bytes;
    }
    return rs.status;
  }
}

int DaemonClient::release(const std::string& key) {
  DaemonRequest rq;
  rq.op = kOpRelease;
  rq.worker = worker_;
  rq.epoch = epoch_;
  set_key(rq.key, key);
  DaemonResponse rs;
  if (!roundtrip(rq, &rs)) return -100;
  return rs.status;
}

}  // namespace bgcore

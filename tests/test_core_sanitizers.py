"""The host-side native engine under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer.

A driver compiled here with g++ links the engine's CUDA-free sources (host paged KV + prefix coordinator, weight slot
table) with the sanitizer runtimes and walks them through allocation, sharing, prefix commit / lookup / eviction,
attach from a second mapping, and a four-thread allocate / free / commit stress.  Any report fails the test."""
import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "batchgen_b200", "core", "csrc")

DRIVER = r"""
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>
#include "host_kv.h"
#include "weight_slot_table.h"
using bgcore::HostPagedKV;

static void key_of(uint8_t* k, int a, int b) { std::memset(k, 0, 32); std::memcpy(k, &a, 4); std::memcpy(k + 4, &b, 4); }

static int worker(HostPagedKV* kv, int tid, int rounds) {
  int bad = 0;
  std::vector<int32_t> pages(8);
  uint8_t keys[4 * 32];
  for (int r = 0; r < rounds; ++r) {
    if (!kv->alloc(8, pages.data())) { kv->prefix_evict(8); continue; }
    for (int i = 0; i < 8; ++i) std::memset(kv->page_ptr(pages[i]), tid, kv->page_bytes());
    for (int i = 0; i < 4; ++i) key_of(keys + 32 * i, tid, r * 4 + i);
    kv->prefix_commit(keys, pages.data(), 4);
    kv->share(pages.data() + 4, 2);
    kv->free_pages(pages.data() + 4, 2);
    int32_t got[4];
    int m = kv->prefix_lookup_attach(keys, 4, got);
    if (m > 0) kv->free_pages(got, m);
    kv->free_pages(pages.data(), 8);
    for (int i = 4; i < 8; ++i) bad += kv->refcount(pages[i]) < 0;
  }
  return bad;
}

int main() {
  HostPagedKV kv;
  int fd = kv.create(256, 4096, 512);
  if (fd < 0) return 2;
  HostPagedKV other;                       // a second mapping of the same region (what a worker does)
  if (!other.attach(fd)) return 3;
  int32_t p[3];
  if (!kv.alloc(3, p)) return 4;
  std::memset(other.page_ptr(p[1]), 0x5a, other.page_bytes());
  if (static_cast<uint8_t*>(kv.page_ptr(p[1]))[4095] != 0x5a) return 5;
  kv.free_pages(p, 3);
  std::vector<std::thread> ts;
  std::vector<int> bad(4, 0);
  for (int t = 0; t < 4; ++t) ts.emplace_back([&, t] { bad[t] = worker(t % 2 ? &kv : &other, t, 300); });
  for (auto& t : ts) t.join();
  for (int b : bad) if (b) return 6;
  kv.prefix_clear();
  if (kv.audit() != 0) return 7;
  if (kv.num_free() != kv.num_pages()) return 8;
  other.detach();
  std::puts("ok");
  return 0;
}
"""


@pytest.mark.parametrize("flags", [["-fsanitize=address,undefined", "-fno-sanitize-recover=all"], ["-fsanitize=thread"]],
                         ids=["asan-ubsan", "tsan"])
def test_host_engine_under_sanitizers(tmp_path, flags):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    src = tmp_path / "driver.cpp"
    src.write_text(DRIVER)
    exe = tmp_path / "driver"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, f"-I{CSRC}", str(src),
           os.path.join(CSRC, "host_kv.cpp"), "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip("sanitizer runtime not installed: " + build.stderr.splitlines()[-1])
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=300)
    assert run.returncode == 0 and "ok" in run.stdout, (run.returncode, run.stdout[-500:], run.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in run.stderr and "WARNING: ThreadSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr


DAEMON_DRIVER = r"""
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
#include <unistd.h>
#include "host_kv_views.h"
#include "weight_daemon.h"
using namespace bgcore;

int main(int argc, char** argv) {
  const std::string dir = argv[1];
  const int port0 = std::atoi(argv[2]), port1 = std::atoi(argv[3]);
  const int n_mod = 8;
  const uint64_t mb = 2048;
  std::vector<std::string> keys;
  for (int i = 0; i < n_mod; ++i) keys.push_back("layer" + std::to_string(i));
  std::vector<uint8_t> store[2];
  for (int node = 0; node < 2; ++node) {
    store[node].resize(mb * n_mod / 2);
    for (int j = 0; j < n_mod / 2; ++j) std::memset(store[node].data() + j * mb, 2 * j + node + 1, mb);
  }
  std::vector<WeightDaemon*> ds;
  for (int node = 0; node < 2; ++node) {
    DaemonConfig c;
    c.node = node;
    c.socket_path = dir + "/wd" + std::to_string(node) + ".sock";
    c.listen_port = node ? port1 : port0;
    c.peers[1 - node] = "127.0.0.1:" + std::to_string(node ? port0 : port1);
    c.staging_slots = 3;
    c.slot_bytes = mb;
    auto* d = new WeightDaemon(c);
    d->set_local_store(store[node].data(), store[node].size());
    for (int i = 0; i < n_mod; ++i) d->add_module(keys[i], i % 2, (uint64_t)(i / 2) * mb, mb);
    d->set_schedule(keys);
    ds.push_back(d);
  }
  for (auto* d : ds) if (!d->start()) return 2;
  int bad = 0;
  auto worker = [&](int node, int id) {
    DaemonClient cl;
    if (!cl.connect_to(dir + "/wd" + std::to_string(node) + ".sock") || cl.hello(id, ds[node]->epoch()) != 0) { bad++; return; }
    for (int sweep = 0; sweep < 3; ++sweep)
      for (int i = 0; i < n_mod; ++i) {
        int slot = -1; uint64_t off = 0, by = 0;
        if (cl.acquire(keys[i], 20000, &slot, &off, &by) != 0 || by != mb) { bad++; return; }
        if ((slot < 0) != (i % 2 == node)) bad++;
        cl.release(keys[i]);
      }
  };
  std::vector<std::thread> ts;
  for (int node = 0; node < 2; ++node) for (int w = 0; w < 2; ++w) ts.emplace_back(worker, node, w);
  for (auto& t : ts) t.join();
  ds[0]->begin_swap();
  const std::string rep = ds[0]->finish_swap();
  if (rep.find("\"ok\": true") == std::string::npos) bad++;
  const std::string st = ds[0]->status();
  if (st.find("\"transport_failed\": false") == std::string::npos) bad++;
  for (auto* d : ds) d->stop();
  for (auto* d : ds) delete d;

  // the sequence views over a host region
  HostPagedKV kv;
  if (kv.create(16, 4 * 8 * 2, 0) < 0) return 3;
  SlidingWindowView sw(&kv, 4, 8, 2, 8);
  CompressedRatioView cr(&kv, 4, 8, 2, 4);
  uint8_t row[8] = {1, 2, 3, 4, 5, 6, 7, 8};
  for (size_t pos = 0; pos < 40; ++pos) {
    if (sw.write_rows(1, 0, pos, row, 1) != 1) bad++;
    cr.append(2, 1, pos, row);
  }
  if (sw.active_pages(1) > 3 || cr.stored_tokens(2) != 10) bad++;
  sw.release(1);
  cr.release(2);
  if (kv.num_free() != kv.num_pages() || kv.audit() != 0) bad++;
  if (bad) return 4;
  std::puts("ok");
  return 0;
}
"""


@pytest.mark.parametrize("flags", [["-fsanitize=address,undefined", "-fno-sanitize-recover=all"], ["-fsanitize=thread"]],
                         ids=["asan-ubsan", "tsan"])
def test_weight_daemon_and_views_under_sanitizers(tmp_path, flags):
    """Two node daemons on this host, two worker threads each sweeping the schedule three times, a cohort swap and the
    sequence views, under ASan + UBSan and under TSan."""
    import socket
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    ports = []
    for _ in range(2):
        s = socket.socket(); s.bind(("127.0.0.1", 0)); ports.append(s.getsockname()[1]); s.close()
    src = tmp_path / "daemon_driver.cpp"
    src.write_text(DAEMON_DRIVER)
    exe = tmp_path / "daemon_driver"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, f"-I{CSRC}", str(src),
           os.path.join(CSRC, "host_kv.cpp"), os.path.join(CSRC, "host_kv_views.cpp"), os.path.join(CSRC, "weight_daemon.cpp"),
           "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip("sanitizer runtime not installed: " + build.stderr.splitlines()[-1])
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([str(exe), str(tmp_path), str(ports[0]), str(ports[1])], capture_output=True, text=True, env=env,
                         timeout=300)
    assert run.returncode == 0 and "ok" in run.stdout, (run.returncode, run.stdout[-500:], run.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in run.stderr and "WARNING: ThreadSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr

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

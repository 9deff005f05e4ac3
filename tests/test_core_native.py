"""Native engine on CPU: slot table (compiled standalone with g++), weight ring with the host copy backend,
node-shared host KV + prefix coordinator across processes, CPU GQA decode kernel."""
import multiprocessing as mp
import os
import subprocess
import sys
import time

import pytest
import torch

from batchgen_b200.core import native
from batchgen_b200.ops import ref

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "batchgen_b200", "core", "csrc")

SLOT_TABLE_TEST = r'''
#include "weight_slot_table.h"
#include <cassert>
#include <cstdio>
using namespace bgcore;
int main() {
  WeightSlotTable t(2);
  t.install_queue({10, 11, 12});
  Production p;
  assert(!t.next_production(&p));                 // no open pass
  assert(t.begin_pass(true) == 1);
  assert(t.next_production(&p) && p.module == 10 && p.slot == 0);
  assert(t.next_production(&p) && p.module == 11 && p.slot == 1);
  assert(!t.next_production(&p));                 // ring full
  assert(t.acquire(10) == -1);                    // still FILLING
  t.landed(0);
  assert(t.acquire(11) == -2);                    // out of order
  int s = t.acquire(10);
  assert(s == 0 && t.slot(0).state == SlotState::LEASED);
  t.release(0, true);
  assert(t.slot(0).state == SlotState::PENDING_RELEASE && !t.next_production(&p));
  t.reclaim(0);
  assert(t.next_production(&p) && p.module == 12 && p.slot == 0);
  // carry: the next pass may be produced as soon as this one is fully produced
  assert(t.begin_pass(false) == 2 && t.begin_pass(false) == 0);   // at most two open
  t.landed(1); assert(t.acquire(11) == 1); t.release(1, false);
  assert(t.next_production(&p) && p.module == 10 && p.pass == 2);
  t.landed(0); assert(t.acquire(12) == 0); t.release(0, false);
  assert(t.end_pass());
  // skips: module 11 is idle in pass 2
  t.skip_modules({11});
  t.landed(1); assert(t.acquire(10) == 1); t.release(1, false);
  assert(t.next_production(&p) && p.module == 12);
  assert(t.expected_module() == 12);
  t.landed(p.slot); assert(t.acquire(12) == p.slot); t.release(p.slot, false);
  assert(t.end_pass() && t.skipped_total() == 1);
  // abort: in-flight slots return to FREE when they land
  t.begin_pass(false);
  assert(t.next_production(&p));
  t.abort_all();
  assert(t.slot(p.slot).state == SlotState::FILLING);
  t.landed(p.slot);
  assert(t.slot(p.slot).state == SlotState::FREE && t.count(SlotState::FREE) == 2 && t.open_passes() == 0);
  std::puts("slot table ok");
  return 0;
}
'''


def test_weight_slot_table_standalone(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text(SLOT_TABLE_TEST)
    exe = tmp_path / "t"
    subprocess.run(["g++", "-std=c++17", "-O1", f"-I{CSRC}", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, stdout=subprocess.PIPE, text=True).stdout
    assert "slot table ok" in out


def test_weight_ring_streams_modules_in_order_with_skips():
    ring = native.WeightRing(num_slots=3, slot_bytes=1 << 16, device="cpu")
    mods = {}
    for i in range(8):
        mods[f"expert_{i}"] = {"w13": torch.full((16, 32), float(i)), "w2": torch.full((8, 16), float(-i)).bfloat16()}
        ring.register(f"expert_{i}", mods[f"expert_{i}"])
    order = [f"expert_{i}" for i in range(8)]
    ring.install_queue(order)
    ring.start()
    for p in range(3):
        assert ring.begin_pass(carry=True) > 0
        skipped = ["expert_3", "expert_6"] if p == 1 else []
        ring.skip(skipped)
        for k in order:
            if k in skipped:
                continue
            w = ring.get(k, timeout_ms=5000)
            assert w is not None, k
            assert torch.equal(w["w13"], mods[k]["w13"]) and torch.equal(w["w2"], mods[k]["w2"])
            ring.release(k)
        assert ring.end_pass()
    st = ring.stats()
    assert st["modules_copied"] == 22 and st["modules_skipped"] == 2 and st["stalls"] == 0
    # out-of-order request and stall bound
    ring.begin_pass()
    assert ring.get("expert_5", timeout_ms=50) is None
    ring.abort()
    ring.stop()
    assert ring.count("LEASED") == 0
    with pytest.raises(ValueError):
        ring.register("huge", {"w": torch.zeros(1 << 20)})
    ring.close()


def _child_attach(fd, q):
    kv = native.HostPagedKV(fd=fd, page_bytes=4096)
    pages = kv.alloc(3)
    kv.page_tensor(pages[0])[:4] = torch.tensor([9, 8, 7, 6], dtype=torch.uint8)
    hit = kv.prefix_lookup_attach(list(range(64)) + [1], 16)
    q.put((pages, hit, kv.num_free))


def test_host_kv_is_shared_between_processes_and_prefix_coordinator_works():
    kv = native.HostPagedKV(num_pages=32, page_bytes=4096, prefix_slots=256)
    assert kv.num_free == 32 and kv.audit() == 0
    mine = kv.alloc(4)
    toks = list(range(64))
    assert kv.prefix_commit(toks, mine, 16) == 4              # 4 full pages published
    assert kv.prefix_commit(toks, mine, 16) == 0              # idempotent
    assert all(kv.refcount(p) == 2 for p in mine)
    ctx = mp.get_context("fork")
    q = ctx.Queue()
    p = ctx.Process(target=_child_attach, args=(kv.fd, q))
    p.start()
    pages, hit, free_in_child = q.get(timeout=30)
    p.join()
    assert hit == mine and set(pages).isdisjoint(mine)
    assert kv.page_tensor(pages[0])[:4].tolist() == [9, 8, 7, 6]       # the child's write is visible here
    assert kv.num_free == 32 - 4 - 3 and all(kv.refcount(p) == 3 for p in mine)
    kv.free(hit)                                                        # the child's references
    kv.free(mine)                                                       # the owner's references: cache keeps them
    assert kv.num_free == 32 - 4 - 3 and kv.prefix_evict(2) == 2        # LRU leaves first
    assert kv.prefix_lookup_attach(toks + [0], 16) == mine[:2]
    kv.free(mine[:2])
    assert kv.prefix_clear() == 2 and kv.num_free == 32 - 3
    kv.free(pages)
    assert kv.num_free == 32 and kv.audit() == 0
    assert kv.alloc(33) is None
    st = kv.prefix_stats()
    assert st["hits"] == 2 and st["evicted"] == 2
    kv.close()


def test_cpu_gqa_decode_matches_reference():
    torch.manual_seed(0)
    B, Hq, Hkv, D, S = 3, 8, 2, 64, 16
    lens = [5, 40, 33]
    q = torch.randn(B, Hq, D)
    ks, vs, kp, vp = [], [], [], []
    for L in lens:
        n = (L + S - 1) // S
        k = torch.randn(n, S, Hkv, D).bfloat16()
        v = torch.randn(n, S, Hkv, D).bfloat16()
        ks.append(k); vs.append(v)
        kp.append([k[i].data_ptr() for i in range(n)]); vp.append([v[i].data_ptr() for i in range(n)])
    for window in (0, 16):
        out = native.cpu_gqa_decode(q, kp, vp, lens, S, Hkv, D ** -0.5, window=window, threads=4)
        for b, L in enumerate(lens):
            k = ks[b].reshape(-1, Hkv, D)[:L].float()
            v = vs[b].reshape(-1, Hkv, D)[:L].float()
            want = ref.gqa_attention(q[b:b + 1], k, v, D ** -0.5, q_start=L - 1, window=window)[0]
            assert torch.allclose(out[b], want, atol=2e-4, rtol=1e-3), (b, window)


def test_parameter_store_loads_converted_checkpoint_and_shares_it(tmp_path):
    import multiprocessing as mp

    import torch

    from batchgen_b200.ckpt import converter
    from batchgen_b200.core.native import ParameterStore
    g = torch.Generator().manual_seed(0)
    shards = {"a": {"w1": torch.randn(33, 7, generator=g), "w2": torch.arange(10, dtype=torch.int32)},
              "b": {"w3": torch.randn(5, 5, generator=g).to(torch.bfloat16)}}
    out = tmp_path / "conv"
    for name, tensors in shards.items():
        converter.convert_shard(str(tmp_path / f"{name}.pt"), str(out), tensors=tensors)
    store = ParameterStore(ParameterStore.bytes_needed(str(out)) + 4096)
    assert store.load_converted(str(out), threads=3) > 0
    for tensors in shards.values():
        for k, v in tensors.items():
            assert torch.equal(store.tensor(k), v)
    idx = store.export_index()
    ctx = mp.get_context("fork")
    q = ctx.Queue()

    def child():
        w = ParameterStore(fd=store.fd, read_only=True)
        w.import_index(idx)
        q.put(float(w.tensor("w1").sum()))
        w.close()

    p = ctx.Process(target=child)
    p.start()
    assert abs(q.get(timeout=20) - float(shards["a"]["w1"].sum())) < 1e-4
    p.join(20)
    store.close()


def test_replica_control_block_barriers_and_abort():
    import threading

    from batchgen_b200.core.native import ParameterStore, ReplicaControlBlock
    store = ParameterStore(ReplicaControlBlock.size() + 4096)
    owner = ReplicaControlBlock(store, 0, members=3, init=True)
    readers = [ReplicaControlBlock(store, 0, members=3, init=False) for _ in range(2)]
    assert readers[0].wait_published(0, 1, frame=1, timeout_ms=30) == ReplicaControlBlock.TIMEOUT
    got = []

    def reader(i):
        rc = readers[i - 1].wait_published(0, 1, frame=1, timeout_ms=5000)
        got.append((i, rc, readers[i - 1].slot_frame(0, 4)))
        readers[i - 1].ack_pulled(i, 1, 1)

    ts = [threading.Thread(target=reader, args=(i,)) for i in (1, 2)]
    [t.start() for t in ts]
    owner.publish(0, 1, slot=4, frame=1)
    assert owner.wait_all_pulled(0, 1, frame=1, timeout_ms=5000) == ReplicaControlBlock.OK
    [t.join() for t in ts]
    assert sorted(got) == [(1, 0, 1), (2, 0, 1)]
    assert owner.wait_all_pulled(0, 1, frame=2, timeout_ms=30) == ReplicaControlBlock.TIMEOUT
    readers[1].abort(2)                                           # a member leaves: waits end at once, by name
    assert owner.wait_all_pulled(0, 1, frame=2, timeout_ms=5000) == ReplicaControlBlock.ABORTED
    store.close()


def test_streamed_experts_match_resident_model_on_cpu():
    """Routed experts kept in host memory and streamed through the native ring give the same logits."""
    import torch

    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.transformer import AttnMeta
    from batchgen_b200.runtime.kv_cache import PagedKVCache
    cfg = get_model_config("tiny-deepseek-v3", num_layers=4, first_k_dense=1)
    T = 20
    ids = torch.arange(T, dtype=torch.int32) % cfg.vocab_size

    def run(model):
        kv = PagedKVCache(cfg, 4, 16, "cpu", torch.float32)
        meta = AttnMeta(mode="prefill", positions=torch.arange(T, dtype=torch.int32), slot_mapping=torch.arange(T, dtype=torch.int64),
                        block_table=torch.arange(2, dtype=torch.int32).view(1, 2), cu_seqlens=[0, T], ctx_lens=[0])
        return model.forward(ids, meta, kv)

    resident = run(build_model(cfg, "cpu", "fp32", seed=0))
    streamed_model = build_model(cfg, "cpu", "fp32", seed=0, stream_experts=True, ring_slots=2)
    assert all(lw.experts is None for lw in streamed_model.w.layers)
    a = run(streamed_model)
    b = run(streamed_model)                                   # a second pass re-streams every layer
    assert torch.equal(a, resident) and torch.equal(b, resident)
    st = streamed_model.streamer.stats()
    assert st["modules_copied"] == 2 * 3 and st["bytes_copied"] == 2 * streamed_model.streamer.bytes_per_pass
    streamed_model.streamer.close()


def test_sliding_window_host_view_keeps_only_the_window_pages():
    from batchgen_b200.core.native import SlidingWindowHostView
    page_tokens, layers, D, window = 4, 2, 8, 8
    kv = native.HostPagedKV(num_pages=6, page_bytes=layers * page_tokens * D * 4, prefix_slots=0)
    view = SlidingWindowHostView(kv, page_tokens, layers, (D,), torch.float32, window)
    rows = torch.arange(40 * D, dtype=torch.float32).view(40, D)
    # a 10-token prefill: positions 0 .. 9, window 8 -> first needed token 2 -> page 0 is still kept
    assert view.write(7, 0, 0, rows[:10].contiguous()) == 10
    assert view.write(7, 1, 0, (rows[:10] + 1000).contiguous()) == 10
    assert view.active_pages(7) == 3 and view.window_start(7) == 0
    got, first = view.read(7, 0)
    assert first == 2 and torch.equal(got, rows[2:10])
    # decode appends: the window start moves page by page and old pages return to the region
    for pos in range(10, 30):
        sp = view.append_position(7, pos)
        assert sp == pos - view.window_start(7)
        view.write(7, 0, pos, rows[pos: pos + 1].contiguous())
        view.write(7, 1, pos, (rows[pos: pos + 1] + 1000).contiguous())
        assert view.active_pages(7) <= window // page_tokens + 1
    assert view.window_start(7) == 20 and kv.num_free == 6 - view.active_pages(7)
    got, first = view.read(7, 1)
    assert first == 22 and torch.equal(got, rows[22:30] + 1000)
    with pytest.raises(IndexError):
        view.write(7, 0, 3, rows[3:5].contiguous())           # older than the kept window
    # a second sequence, then the region runs out
    assert view.write(8, 0, 0, rows[:12].contiguous()) == 8      # positions 0 .. 3 are outside the window already
    assert view.active_pages(8) == 2 and view.window_start(8) == 4
    with pytest.raises(MemoryError):
        view.write(9, 0, 0, rows[:8].contiguous())
    view.release(7); view.release(8); view.release(9)
    assert kv.num_free == 6 and kv.audit() == 0
    with pytest.raises(ValueError):
        SlidingWindowHostView(kv, page_tokens, layers, (D,), torch.float32, 6)     # not a multiple of the page
    view.close(); kv.close()


def test_compressed_ratio_host_view_stores_one_row_per_group():
    from batchgen_b200.core.native import CompressedRatioHostView
    page_tokens, layers, D, ratio = 4, 1, 6, 4
    kv = native.HostPagedKV(num_pages=4, page_bytes=layers * page_tokens * D * 2, prefix_slots=0)
    view = CompressedRatioHostView(kv, page_tokens, layers, (D,), torch.bfloat16, ratio)
    pooled = torch.randn(16, D).to(torch.bfloat16)
    # prefill of 14 raw tokens -> 3 stored rows in one page
    assert view.offload(3, 0, 14, pooled[:3].contiguous()) == 3
    assert view.stored(3) == 3 and view.pages(3) == 1
    # decode: positions 14, 15 -> the row of group 3 is stored at position 15 only
    assert view.append(3, 0, 14, pooled[3]) == -1 and view.stored(3) == 3
    assert view.append(3, 0, 15, pooled[3]) == 3 and view.stored(3) == 4
    for pos in range(16, 24):
        sp = view.append(3, 0, pos, pooled[pos // ratio])
        assert sp == (pos // ratio if (pos + 1) % ratio == 0 else -1)
    assert view.stored(3) == 6 and view.pages(3) == 2
    assert torch.equal(view.read(3, 0), pooled[:6])
    # a sequence shorter than one group holds a page (capacity for its first row) and no rows
    assert view.offload(4, 0, 3, pooled[:1].contiguous()) == 0 and view.stored(4) == 0 and view.pages(4) == 1
    view.release(3); view.release(4)
    assert kv.num_free == 4 and kv.audit() == 0
    view.close(); kv.close()


def _two_daemons(tmp_path, slots=3, depth=2, n_mod=8, mod_bytes=4096):
    """Two nodes on this host: even modules live on node 0, odd ones on node 1; the schedule visits them in order."""
    import socket
    ports = []
    for _ in range(2):
        s = socket.socket(); s.bind(("127.0.0.1", 0)); ports.append(s.getsockname()[1]); s.close()
    keys = [f"layer{i}.experts" for i in range(n_mod)]
    g = torch.Generator().manual_seed(0)
    data = {k: torch.randint(0, 256, (mod_bytes,), generator=g, dtype=torch.uint8) for k in keys}
    daemons = []
    for node in range(2):
        d = native.WeightDaemon(node, str(tmp_path / f"wd{node}.sock"), listen_port=ports[node],
                                peers={1 - node: f"127.0.0.1:{ports[1 - node]}"}, staging_slots=slots,
                                slot_bytes=mod_bytes, prefetch_depth=depth, acquire_wait_ms=50)
        mine = [k for i, k in enumerate(keys) if i % 2 == node]
        d.set_local_store(torch.cat([data[k] for k in mine]))
        for i, k in enumerate(keys):
            d.add_module(k, i % 2, (i // 2) * mod_bytes, mod_bytes)
        d.set_schedule(keys)
        daemons.append(d)
    for d in daemons:
        d.start()
    return daemons, keys, data


def test_weight_daemon_serves_local_and_remote_modules_with_prefetch(tmp_path):
    daemons, keys, data = _two_daemons(tmp_path)
    try:
        d0 = daemons[0]
        c = native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch)
        staging = d0.staging()
        for sweep in range(2):                                   # the schedule is cyclic
            for i, k in enumerate(keys):
                where, off, nb = c.acquire(k, timeout_ms=20_000)
                assert nb == 4096 and where == ("local" if i % 2 == 0 else "staging")
                src = d0._store if where == "local" else staging
                assert torch.equal(src[off: off + nb], data[k]), k
                c.release(k)
        st = d0.status()
        assert st["acquires"] == 16 and st["local"] == 8 and st["fetches"] >= 4
        assert st["ready_hits"] >= 1                              # prefetch ran ahead of the worker at least once
        assert st["transport_failed"] is False and st["fetch_ms"]["count"] == st["fetches"]
        served = daemons[1].status()["bytes_served"]             # a prefetch may be in flight between the two reads
        assert st["bytes_fetched"] <= served <= st["bytes_fetched"] + 3 * 4096   # at most the staging slots
        c.close()
    finally:
        for d in daemons:
            d.stop()


def test_weight_daemon_leases_retry_and_cohort_swap(tmp_path):
    daemons, keys, data = _two_daemons(tmp_path, slots=2, depth=1)
    try:
        d0 = daemons[0]
        with pytest.raises(PermissionError):
            native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch + 1)      # wrong cohort epoch
        a = native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch)
        b = native.WeightDaemonClient(d0.socket_path, worker=1, epoch=d0.epoch)
        assert a.acquire(keys[1], 20_000)[0] == "staging"
        assert b.acquire(keys[3], 20_000)[0] == "staging"
        # both slots are leased: a third remote module cannot become ready
        with pytest.raises(TimeoutError):
            a.acquire(keys[5], timeout_ms=300)
        assert d0.status()["retries"] >= 1
        b.close()                                                  # a closed connection gives its lease back
        assert a.acquire(keys[5], 20_000)[0] == "staging"
        with pytest.raises(RuntimeError):
            a.acquire("no.such.module", 1000)
        # cohort swap: the open cohort is cut off, everything is released, the next epoch is admitted
        a2 = native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch)
        assert a2.acquire(keys[1], 20_000)[0] == "staging"         # shares the ready slot
        old = d0.begin_swap()
        with pytest.raises(PermissionError):
            native.WeightDaemonClient(d0.socket_path, worker=2, epoch=old)
        with pytest.raises(RuntimeError):
            a2.acquire(keys[3], 1000)
        report = d0.finish_swap()
        assert report["ok"] and report["epoch"] == old + 1 and report["leases_released"] >= 1
        assert d0.status()["slots"]["leased"] == 0 and d0.status()["cursor"] == 0
        c = native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch)
        where, off, nb = c.acquire(keys[1], 20_000)
        assert where == "staging" and torch.equal(d0.staging()[off: off + nb], data[keys[1]])
        c.close(); a2.close()
    finally:
        for d in daemons:
            d.stop()


def test_weight_daemon_latches_a_transport_failure(tmp_path):
    daemons, keys, data = _two_daemons(tmp_path)
    try:
        d0, d1 = daemons
        c = native.WeightDaemonClient(d0.socket_path, worker=0, epoch=d0.epoch)
        assert c.acquire(keys[1], 20_000)[0] == "staging"
        c.release(keys[1])
        d1.stop()                                                  # the owning node goes away
        with pytest.raises((RuntimeError, TimeoutError)):
            for k in keys[1::2] * 3:
                c.acquire(k, 3000)
                c.release(k)
        for _ in range(100):
            if d0.status()["transport_failed"]:
                break
            time.sleep(0.1)
        st = d0.status()
        assert st["transport_failed"] and "failed" in st["cohort_fault"]
        c2 = native.WeightDaemonClient(d0.socket_path, worker=1, epoch=d0.epoch)
        assert c2.acquire(keys[0], 1000)[0] == "local"             # local modules are still served
        with pytest.raises(RuntimeError):
            c2.acquire(keys[7], 1000)
    finally:
        for d in daemons:
            d.stop()


def test_distributed_module_source_reads_local_and_remote_modules(tmp_path):
    daemons, keys, data = _two_daemons(tmp_path)
    try:
        d1 = daemons[1]
        client = native.WeightDaemonClient(d1.socket_path, worker=0, epoch=d1.epoch)
        src = native.DistributedModuleSource(d1._store, d1.staging(), client)
        for k in keys:
            t = src.tensor(k, torch.int16, (2048,))
            assert torch.equal(t.view(torch.uint8), data[k]), k
        assert src.local_reads == 4 and src.remote_reads == 4
        assert d1.status()["slots"]["leased"] == 0               # every lease went back
        client.close()
    finally:
        for d in daemons:
            d.stop()


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_slot_kv_storage_with_heterogeneous_decode_attention(mode):
    """Slot-based host KV: decode attention on the host kernel (mode 1), through the double-buffered device copy
    (mode 0, on CPU tensors here) and split between both (mode 2) equals the reference attention over the same rows."""
    from batchgen_b200.runtime.hetero_attention import HeteroAttention, SlotKVStorage
    torch.manual_seed(1)
    layers, Hq, Hkv, D = 2, 8, 2, 64
    st = SlotKVStorage(layers, slots=4, max_len=48, num_kv_heads=Hkv, head_dim=D)
    lens = [5, 40, 33]
    slots = [st.acquire() for _ in lens]
    kv = {}
    for l in range(layers):
        for s, L in zip(slots, lens):
            k, v = torch.randn(L, Hkv, D), torch.randn(L, Hkv, D)
            st.write(l, s, 0, k[: L - 1], v[: L - 1])           # the prompt ...
            st.write(l, s, L - 1, k[L - 1:], v[L - 1:])         # ... and the decoded token
            kv[(l, s)] = (k.bfloat16().float(), v.bfloat16().float())
    assert [st.lens[s] for s in slots] == lens and st.num_free == 1
    att = HeteroAttention(st, Hq, mode=mode, device="cpu", host_fraction=0.5, threads=4, max_batch=4)
    for l in range(layers):
        if mode != 1 and l + 1 < layers:
            att.prefetch(l + 1, slots, lens)                    # the next layer streams in while this one computes
        q = torch.randn(len(lens), Hq, D)
        for window in (0, 16):
            out = att.decode(l, q, slots, lens, window=window)
            for b, (s, L) in enumerate(zip(slots, lens)):
                k, v = kv[(l, s)]
                want = ref.gqa_attention(q[b:b + 1], k, v, D ** -0.5, q_start=L - 1, window=window)[0]
                assert torch.allclose(out[b], want, atol=2e-4, rtol=1e-3), (mode, l, b, window)
    if mode == 2:
        assert att.host_rows > 0 and att.device_rows > 0
    with pytest.raises(ValueError):
        st.write(0, slots[0], 47, torch.zeros(2, Hkv, D), torch.zeros(2, Hkv, D))
    for s in slots:
        st.release(s)
    assert st.num_free == 4

"""Pure policy modules: continuous batching, decode DP groups, weight replica planning."""
import pytest

from batchgen_b200.core import weight_replica as wr
from batchgen_b200.parallel import dp_groups as dg
from batchgen_b200.runtime import continuous_batching as cb


def test_adaptive_chunk_sizer_follows_ema():
    s = cb.AdaptiveChunkSizer(initial_chunk=8192, min_chunk=1024, max_chunk=65536)
    for _ in range(9):
        s.report_completion(1000)
    assert s.get_chunk_size() == 8192                     # not enough samples yet
    s.report_completion(1000)
    assert s.get_chunk_size() == 1536                     # 1.5 x 1000 rounded up to a page
    for _ in range(200):
        s.report_completion(100000)
    assert s.get_chunk_size() == 65536                    # clamped
    assert s.get_chunk_size() % 64 == 0


def test_eviction_selection_is_deterministic_and_priority_aware():
    seqs = [("b", {"decoded_length": 5, "gpu_pages_allocated": 2}), ("a", {"decoded_length": 5, "gpu_pages_allocated": 2}),
            ("c", {"decoded_length": 1, "gpu_pages_allocated": 3, "priority": 1}),
            ("d", {"decoded_length": 9, "gpu_pages_allocated": 4})]
    v, freed = cb.select_sequences_for_eviction(seqs, 4)
    assert v == ["a", "b"] and freed == 4                 # high-priority 'c' is spared, ties by uuid
    v, _ = cb.select_sequences_for_eviction(seqs, 3, cb.EvictionStrategy.LONGEST_FIRST)
    assert v == ["d"]
    with pytest.raises(ValueError):
        cb.select_sequences_for_eviction(seqs, 1, cb.EvictionStrategy.GROWTH_COST_AWARE)


def test_growth_evictions_are_growth_driven():
    cands = [("s1", {"decoded_length": 10, "host_owned_pages": 4, "global_idx": 1, "growth_pages": 2, "recompute_tokens": 1000}),
             ("s2", {"decoded_length": 50, "host_owned_pages": 8, "global_idx": 2, "growth_pages": 2, "recompute_tokens": 400}),
             ("s3", {"decoded_length": 70, "host_owned_pages": 2, "global_idx": 3, "growth_pages": 2, "recompute_tokens": 5000})]
    common = dict(active_uuids=["s1", "s2", "s3"], completed_uuids=[], host_growth_uuids=["s1", "s2", "s3"],
                  host_growth_pages=[2, 2, 2], eviction_candidates=cands, total_pages=100, completed_pages=0)
    # a full pool with enough free pages for the debt evicts nobody
    p = cb.plan_host_kv_growth_evictions(free_pages=6, **common)
    assert p.evicted_uuids == [] and p.growth_feasible_after_eviction
    # debt 6, free 1: shortest-first evicts s1 (returns 4 pages and retires 2 of debt) -> 5 free >= 4 needed
    p = cb.plan_host_kv_growth_evictions(free_pages=1, **common)
    assert p.evicted_uuids == ["s1"] and p.remaining_growth_needed == 4 and p.expected_free_pages == 5
    # cost-aware: s2 closes 10 deficit pages for 400 recompute tokens -> best ratio
    p = cb.plan_host_kv_growth_evictions(free_pages=1, strategy=cb.EvictionStrategy.GROWTH_COST_AWARE, **common)
    assert p.evicted_uuids == ["s2"]
    # reclaimable prefix pages count as supply
    p = cb.plan_host_kv_growth_evictions(free_pages=1, reclaimable_pages=5, **common)
    assert p.evicted_uuids == []


def test_loading_selection_respects_buckets_and_slots():
    cands = {"a": {"decoded_length": 9, "pages_needed": 4, "assigned_rank": 0},
             "b": {"decoded_length": 7, "pages_needed": 4, "assigned_rank": 0},
             "c": {"decoded_length": 5, "pages_needed": 1, "assigned_rank": 1}}
    got, used = cb.select_sequences_for_loading(cands, [6, 1], set())
    assert got == ["a", "c"] and used == {0: 4, 1: 1}
    got, _ = cb.select_sequences_for_loading(cands, [8, 1], {"a"}, per_group_seq_slots=[1, 0])
    assert got == ["b"]
    grouped = {"x": {"decoded_length": 3, "pages_needed": 2, "decode_dp_group": 1}}
    got, used = cb.select_sequences_for_loading(grouped, [9, 9, 2, 5], set(), group_size=2)
    assert got == ["x"] and used[1] == 2                  # capacity of group 1 = min(2, 5)
    with pytest.raises(ValueError):
        cb.select_sequences_for_loading(grouped, [1, 2, 3], set(), group_size=2)


def test_decode_dp_groups():
    assert dg.num_decode_dp_groups(8, 2) == 4
    with pytest.raises(ValueError):
        dg.num_decode_dp_groups(8, 3)
    assert dg.rank_in_decode_group(1, 3, 2) and not dg.rank_in_decode_group(1, 4, 2) and not dg.rank_in_decode_group(None, 0, 2)
    assert dg.host_kv_owner_rank(3, 2) == 6
    groups = dg.assign_decode_dp_groups([100, 10, 90, 20], 2)
    assert groups == [0, 1, 1, 1] or sorted(groups) == [0, 1, 1, 1]
    pinned = dg.assign_decode_dp_groups([100, 10], 2, pinned=[None, 0])
    assert pinned[1] == 0

    class Seq:
        decode_dp_group = 2
    s = Seq()
    dg.evict_from_decode_dp_group(s)
    assert s.decode_dp_group is None and s.evicted_from_dp_group == 2
    dg.evict_from_decode_dp_group(s)
    assert s.evicted_from_dp_group == 2                   # a redundant eviction keeps the record
    assert dg.decode_group_plan_digest([(1, 0), (2, 1)]) == dg.decode_group_plan_digest([(2, 1), (1, 0)])
    assert dg.first_group_disagreement([[(1, 0), (2, 1)], [(1, 0), (2, 0)]]) == (2, [1, 0])
    assert dg.moe_rows_per_rank(33, 8) == 5
    assert dg.decode_group_rows([3, 3, 5, 4], 2) == [3, 5]
    assert dg.count_rows_per_group([0, 1, 1, None], 2) == [1, 2]


def test_weight_replica_plan():
    acc = {r: True for r in range(4)}
    recs = [wr.RankRecord(r, "node0", "fp", acc) for r in range(4)] + [wr.RankRecord(4, "node1", "fp", {}),
                                                                      wr.RankRecord(5, "node0", "fp", {}, "resident")]
    groups = wr.compute_replica_groups(recs)
    assert groups[0] == (0, 1, 2, 3) and groups[4] == (4,) and groups[5] == (5,)
    bad = [wr.RankRecord(0, "n", "f", {1: True}), wr.RankRecord(1, "n", "f", {0: False})]
    with pytest.raises(ValueError):
        wr.compute_replica_groups(bad)
    task = {"attn": [f"attn_{l}" for l in range(3)],
            "routed_expert": [f"routed_expert_{l}_{e}" for l in (1, 2) for e in range(8)]}
    plan = wr.derive_frame_plan(task)
    assert plan.layer_sequence == (0, 1, 2) and plan.frame_size == {"attn": 1, "routed_expert": 8}
    owners = wr.derive_owner_map((0, 1, 2, 3), task, plan)
    assert [owners[f"routed_expert_1_{e}"] for e in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    assert [owners[f"attn_{l}"] for l in range(3)] == [0, 1, 2]
    sizes = {n: (100 if n.startswith("routed") else 10) for names in task.values() for n in names}
    per_rank = wr.bytes_copied_per_rank(owners, sizes)
    assert per_rank[3] == 400 and per_rank[0] == 410
    kinds = wr.record_kinds(1, (0, 1, 2, 3), owners)
    assert kinds["attn_1"] == wr.REPLICA_OWNER and kinds["attn_0"] == wr.REPLICA_READER
    assert set(wr.record_kinds(0, (0,), owners).values()) == {wr.HOST_PRIVATE}
    frames = wr.plan_broadcast_frames(task, plan, owners)
    assert frames[0].frame == 0 and frames[0].modules == ("attn_0",)
    assert [f.frame for f in frames] == sorted(f.frame for f in frames)
    assert wr.derive_frame_plan({"attn": ["attn_2", "attn_1"]}) is None     # out of order
    assert wr.derive_frame_plan({"x": ["weird"]}) is None


def test_owner_layout_blocks_pads_and_keeps_owners():
    """Request-split decode: one block per rank, rows stay with their owner, new rows go to the least loaded rank,
    and the step length is rounded to a captured graph size."""
    import types

    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.sequence import S, Sequence

    seqs = {i: Sequence(global_idx=i, prompt_ids=[1, 2, 3]) for i in range(7)}
    for s in seqs.values():
        s.status = S.IN_DECODE
    eng = types.SimpleNamespace(model=types.SimpleNamespace(layout=types.SimpleNamespace(tp_size=4)), seqs=seqs,
                                graph_runner=None)
    layout = Engine._owner_layout(eng, list(seqs.values()))
    assert len(layout) == 8 and [s.decode_owner for s in seqs.values()] == [0, 1, 2, 3, 0, 1, 2]
    assert [None if s is None else s.global_idx for s in layout] == [0, 4, 1, 5, 2, 6, 3, None]
    # rows 0 and 4 leave; a new row joins the rank that now owns the fewest; nobody else moves
    for i in (0, 4):
        seqs[i].status = S.COMPLETED
    seqs[7] = Sequence(global_idx=7, prompt_ids=[1])
    seqs[7].status = S.IN_DECODE
    live = [s for s in seqs.values() if s.status == S.IN_DECODE]
    before = {s.global_idx: s.decode_owner for s in live if s.decode_owner >= 0}
    layout = Engine._owner_layout(eng, live)
    assert seqs[7].decode_owner == 0 and all(s.decode_owner == o for s in live for g, o in before.items() if s.global_idx == g)
    assert [None if s is None else s.global_idx for s in layout] == [7, None, 1, 5, 2, 6, 3, None]
    # with a graph runner the whole step is one of the captured sizes (a multiple of the group size)
    eng.graph_runner = types.SimpleNamespace(bucketing=types.SimpleNamespace(bucket_for=lambda n: 16))
    assert len(Engine._owner_layout(eng, live)) == 16


def test_state_pool_is_budgeted():
    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.runtime.planner import state_pool_bytes
    cfg = get_model_config("kimi-k3-kda")
    one = state_pool_bytes(cfg, EngineConfig(max_state_slots=1, attn_tp_size=8, world_size=8))
    # 69 layers x 8 heads x (128 x 128 + 9 x 128) fp32
    assert one == 69 * 8 * (128 * 128 + 9 * 128) * 4
    assert state_pool_bytes(cfg, EngineConfig(max_decode_batch=64, attn_tp_size=8, world_size=8)) == 64 * one

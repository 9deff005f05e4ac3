"""Trajectory frontier registry: commit after a turn, restore on the next, named declines, refcounts."""
import pytest

from batchgen_b200.runtime import trajectory as tj


def test_commit_and_restore_roundtrip():
    released = []
    reg = tj.TrajectoryFrontierRegistry(page_tokens=4, page_bytes=100, namespace=(7, 1), release_fn=released.append)
    turn1 = list(range(10))                                   # prompt + generated of the finished turn
    rec = reg.advance("sess", turn1, page_ids=[11, 12, 13], snapshot=tj.StateSnapshot(0, 64, shards=2), owning_group=3)
    assert rec.boundary_tokens == 8 and rec.page_ids == (11, 12) and rec.charge.total_bytes == 2 * 100 + 128
    hit = reg.resolve("sess", turn1 + [50, 51, 52])
    assert hit.hit and hit.boundary_tokens == 8 and hit.record.refcount == 2
    hit.record.release()
    assert reg.resolve("sess", turn1[:8]).reason == tj.DECLINE_PROMPT_TOO_SHORT
    assert reg.resolve("sess", [0, 1, 2, 99] + turn1[4:] + [1]).reason == tj.DECLINE_PROMPT_DIVERGES
    assert reg.resolve("other", turn1 + [1]).reason == tj.DECLINE_NO_SESSION
    assert reg.resolve("sess", turn1 + [1], namespace=(7, 2)).reason == tj.DECLINE_NAMESPACE
    assert reg.session_group_summary()[reg.key("sess")] == (3, 8)
    reg.check_invariants()
    assert reg.stats["hits"] == 1 and reg.stats["declines"] == 4 and not released


def test_advance_replaces_and_old_record_leaves_with_last_reader():
    released = []
    reg = tj.TrajectoryFrontierRegistry(4, 10, release_fn=lambda r: released.append(r.page_ids))
    reg.advance("s", list(range(9)), [1, 2])
    reader = reg.resolve("s", list(range(9)) + [1]).record     # a restore in flight
    reg.advance("s", list(range(13)), [1, 2, 3])               # next turn commits a longer frontier
    assert released == []                                       # the reader still holds the old record
    reader.release()
    assert released == [(1, 2)]
    with pytest.raises(tj.FrontierRefcountError):
        reader.release()
    assert reg.get("s").boundary_tokens == 12 and len(reg) == 1
    assert reg.total_charge().pages == 3


def test_eviction_and_short_trajectories():
    released = []
    reg = tj.TrajectoryFrontierRegistry(4, 10, release_fn=lambda r: released.append(r.session_key))
    with pytest.raises(tj.FrontierRegistryError):
        reg.advance("tiny", [1, 2, 3, 4], [1])                 # the last token must stay private
    for i in range(3):
        reg.advance(f"s{i}", list(range(9)), [10 * i, 10 * i + 1])
    busy = reg.resolve("s0", list(range(9)) + [5]).record
    freed = reg.evict_for_pages(3, ["s0", "s1", "s2"])         # s0 is being read: skipped
    assert freed == 4 and reg.get("s1") is None and reg.get("s2") is None and reg.get("s0") is not None
    busy.release()
    assert reg.evict("s0") is True and len(released) == 3
    with pytest.raises(tj.FrontierRegistryError):
        reg.evict("s0")
    assert tj.aligned_prefix_tokens(8, 4) == 4 and tj.aligned_prefix_tokens(9, 4) == 8

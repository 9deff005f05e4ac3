"""QueryBook: paged token book with up-front reservations, turns and a node-shared backing store."""
import multiprocessing as mp

import pytest
import torch

from batchgen_b200.runtime.query_book import NodeSharedTokens, QueryBook


def test_bind_write_append_release():
    qb = QueryBook(capacity_bytes=16 * 8 * 4, page_tokens=8)           # 16 pages of 8 tokens
    a = qb.bind("a", 20)                                               # 3 pages
    b = qb.bind("b", 8)
    assert qb.free_page_count == 12 and qb.active_count == 2
    qb.write_prompt(a, torch.arange(10))
    for t in (100, 101, 102):
        qb.append_token(a, t)
    assert qb.tokens(a).tolist() == list(range(10)) + [100, 101, 102]
    assert qb.generated_tokens(a).tolist() == [100, 101, 102] and qb.last_generated_token(a) == 102
    turn = qb.turns(a)[0]
    assert (turn.token_start, turn.prompt_end, turn.generated_end) == (0, 10, 13)
    with pytest.raises(ValueError):
        qb.write_prompt(b, torch.arange(9))                            # beyond the reservation
    with pytest.raises(ValueError):
        qb.bind("a", 4)
    qb.release(a)
    assert qb.free_page_count == 15 and not qb.has_sequence("a") and qb.audit() == 0
    c = qb.bind("c", 24)                                               # reuses the freed extent + neighbours
    assert qb.slot_for("c") == c and qb.audit() == 0


def test_all_or_nothing_batches_and_fragmentation():
    qb = QueryBook(capacity_bytes=10 * 4 * 4, page_tokens=4)           # 10 pages
    s = qb.bind_batch(["x", "y", "z"], [8, 4, 12])                    # 2 + 1 + 3 pages
    assert qb.free_page_count == 4
    qb.release(s[0])                                                   # largest first: z=0..2, x=3..4, y=5
    assert qb.free_page_count == 6 and qb.largest_free_extent_pages == 4
    assert not qb.can_reserve(20) and qb.can_reserve(16)
    assert not qb.can_reserve_batch([16, 12])                          # 4 + 3 pages do not fit extents of 2 and 4
    with pytest.raises(MemoryError):
        qb.bind_batch(["p", "q"], [16, 12])
    assert not qb.has_sequence("p") and qb.audit() == 0


def test_turns_and_reentry_and_copy():
    qb = QueryBook(capacity_bytes=64 * 4 * 4, page_tokens=4)
    s = qb.bind("sess", 40)
    qb.write_prompt(s, torch.tensor([1, 2, 3]))
    qb.append_tokens([s, s], [7, 8])
    qb.append_prompt(s, torch.tensor([4, 5]))                          # next turn of an agent session
    qb.append_token(s, 9)
    assert [(t.token_start, t.prompt_end, t.generated_end) for t in qb.turns(s)] == [(0, 3, 5), (5, 7, 8)]
    assert qb.generated_tokens(s).tolist() == [9]
    t = qb.begin_reentry_turn(s, 8)                                    # evicted: everything becomes prompt
    assert (t.token_start, t.prompt_end) == (0, 8)
    with pytest.raises(ValueError):
        qb.begin_reentry_turn(s, 5)
    other = QueryBook(capacity_bytes=64 * 4 * 4, page_tokens=4)
    o = other.bind("sess", 40)
    qb.copy_to(s, other, o)
    assert other.tokens(o).tolist() == qb.tokens(s).tolist() and len(other.turns(o)) == 3


def _child(handle, q):
    shared = NodeSharedTokens.attach(handle)
    q.put(shared.tensor[1, :3].tolist())
    shared.tensor[0, 0] = 4242


def test_node_shared_backing_store():
    shared = NodeSharedTokens.create(rows=4, width=8)
    qb = QueryBook(capacity_bytes=4 * 8 * 4, page_tokens=8, storage=shared.tensor)
    s = qb.bind("a", 8)
    qb.bind("b", 8)
    qb.write_prompt(qb.slot_for("b"), torch.tensor([5, 6, 7]))
    ctx = mp.get_context("fork")
    q = ctx.Queue()
    p = ctx.Process(target=_child, args=(shared.handle(), q))
    p.start()
    assert q.get(timeout=20) == [5, 6, 7]
    p.join(20)
    assert p.exitcode == 0 and int(shared.tensor[0, 0]) == 4242 and s == 0
    shared.release_fd()
    assert int(shared.tensor[1, 0]) == 5                               # the mapping outlives the descriptor

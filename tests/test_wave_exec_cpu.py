"""In-wave prefix sharing executed by the engine, and trajectory restore across turns (CPU, fp32)."""
import random

import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.sequence import SamplingParams


def _engine(prefix: bool, pages: int = 700, **kw):
    cfg = get_model_config("tiny-deepseek-v3")
    model = build_model(cfg, "cpu", "fp32", seed=3)
    return cfg, Engine(model, EngineConfig(page_size=16, enable_prefix_cache=prefix, max_decode_batch=128, **kw),
                       num_gpu_pages=pages)


def test_grouped_prefix_wave_computes_each_prefix_once():
    """8 shared prefixes x 8 suffixes in one wave (the grouped-prefix workload, scaled down): every prefix is
    computed once, every request still produces the tokens it produces without any sharing."""
    cfg, plain = _engine(False)
    rng = random.Random(0)
    P, S, page = 8, 8, 16
    prefixes = [[rng.randrange(2, cfg.vocab_size) for _ in range(5 * page)] for _ in range(P)]
    prompts = [pre + [rng.randrange(2, cfg.vocab_size) for _ in range(7)] for pre in prefixes for _ in range(S)]
    sp = SamplingParams(max_new_tokens=4, ignore_eos=True)
    want = plain.generate(prompts, sp)
    _, eng = _engine(True, pages=300)          # 64 x 7 pages would not fit: admission charges a shared block once
    got = eng.generate(prompts, sp)
    assert got == want
    total = sum(len(p) for p in prompts)
    shared = (S - 1) * P * 5 * page
    assert eng.stats.prefill_waves == 1
    assert eng.stats.prefill_tokens == total - shared                # each prefix once, each tail once
    assert eng.stats.shared_prefix_tokens == shared
    assert eng.stats.prefill_cached_tokens == P * S * 5 * page       # reported per request (usage.cached_tokens)
    # everything a sequence held is released; what stays is held by the prefix cache alone
    held = eng.kv.alloc.num_used
    assert held == eng.prefix.reclaimable_pages()
    eng.prefix.clear()
    assert eng.kv.alloc.num_used == 0


def test_nested_prefixes_and_cross_wave_cache():
    """Two levels of sharing inside a wave (a common head, then two branches), then a second wave that hits the
    pages the first wave left in the cache."""
    cfg, plain = _engine(False)
    rng = random.Random(1)
    tok = lambda n: [rng.randrange(2, cfg.vocab_size) for _ in range(n)]
    head, b1, b2 = tok(32), tok(32), tok(16)
    prompts = [head + b1 + tok(5), head + b1 + tok(9), head + b2 + tok(3), head + b2 + tok(20), head + tok(2), tok(40)]
    sp = SamplingParams(max_new_tokens=3, ignore_eos=True)
    want = plain.generate(prompts, sp)
    _, eng = _engine(True)
    assert eng.generate(prompts, sp) == want
    assert eng.stats.shared_prefix_tokens == 4 * 32 + 32 + 16        # head by 5 (4 saved), b1 and b2 by 2 each
    before = eng.stats.prefill_tokens
    again = [head + b1 + tok(4), tok(33)]
    want2 = plain.generate(again, sp)
    assert eng.generate(again, sp) == want2
    assert eng.stats.prefill_tokens - before == 4 + 33               # head + b1 came from the cache


def test_second_turn_of_a_session_restores_the_first_turns_kv():
    """A finished turn leaves prompt + generated pages in the cache (trajectory commit); the next turn, whose prompt
    extends them, computes only what is new and reports the rest as cached."""
    cfg, plain = _engine(False)
    rng = random.Random(2)
    tok = lambda n: [rng.randrange(2, cfg.vocab_size) for _ in range(n)]
    turn1 = tok(37)
    sp = SamplingParams(max_new_tokens=30, ignore_eos=True)
    _, eng = _engine(True)
    out1 = eng.generate([turn1], sp)[0]
    assert eng.stats.trajectory_commits == 1
    turn2 = turn1 + out1 + tok(6)
    s2 = eng.add_request(turn2, SamplingParams(max_new_tokens=5, ignore_eos=True))
    eng.run_to_completion()
    # 37 + 30 tokens, of which 66 have KV when the turn ends -> 4 full pages of 16 restored
    assert s2.cached_prefix_tokens == 64
    want = plain.generate([turn2], SamplingParams(max_new_tokens=5, ignore_eos=True))[0]
    assert s2.output_ids == want


def test_session_frontier_survives_cache_pressure_until_the_session_ends():
    """A session's last finished turn is pinned (an extra page reference held by its frontier): other requests that
    churn the prefix cache cannot evict it, the next turn restores it, and ending the session releases the pin."""
    cfg, plain = _engine(False)
    rng = random.Random(3)
    tok = lambda n: [rng.randrange(2, cfg.vocab_size) for _ in range(n)]
    sp = SamplingParams(max_new_tokens=12, ignore_eos=True)
    _, eng = _engine(True, pages=40)
    turn1 = tok(52)
    s1 = eng.add_request(turn1, sp, session_id="chat-1")
    eng.run_to_completion()
    assert eng.stats.trajectory_frontiers == 1 and len(eng.trajectories) == 1
    pinned = list(eng.trajectories.get("chat-1").page_ids)               # 52 + 11 cached tokens -> 3 full pages
    assert len(pinned) == 3 and all(eng.kv.alloc.refcount(p) == 2 for p in pinned)
    # unrelated traffic larger than the pool: the cache evicts its own entries, not the pinned pages
    for _ in range(6):
        eng.generate([tok(100)], SamplingParams(max_new_tokens=3, ignore_eos=True))
    assert all(eng.kv.alloc.refcount(p) >= 2 for p in pinned)
    turn2 = turn1 + s1.output_ids + tok(9)
    s2 = eng.add_request(turn2, SamplingParams(max_new_tokens=4, ignore_eos=True), session_id="chat-1")
    eng.run_to_completion()
    assert eng.stats.trajectory_restores == 1 and s2.cached_prefix_tokens == 48
    assert s2.output_ids == plain.generate([turn2], SamplingParams(max_new_tokens=4, ignore_eos=True))[0]
    # the new frontier replaced the old one; a diverging prompt or end_session drops it
    assert eng.stats.trajectory_frontiers == 2 and len(eng.trajectories) == 1
    assert eng.end_session("chat-1") and len(eng.trajectories) == 0 and not eng.end_session("chat-1")
    eng.prefix.clear()
    assert eng.kv.alloc.num_used == 0
    eng.trajectories.check_invariants()

"""In-wave prefix sharing planner and rank packing (pure functions)."""
import random

import pytest

from batchgen_b200.runtime import wave_plan as wp


def _wave(seed=0, block=16):
    rng = random.Random(seed)
    doc = [[rng.randrange(1000) for _ in range(block * 6)] for _ in range(3)]
    prompts = []
    for d in doc:
        for q in range(4):
            prompts.append(d + [rng.randrange(1000) for _ in range(rng.randrange(1, 40))])
    prompts.append([rng.randrange(1000) for _ in range(50)])          # a loner
    prompts.append(doc[0][: block * 3] + [7] * 20)                    # branches off doc 0 half way
    return prompts


def test_plan_accounting_and_order():
    prompts = _wave()
    plan = wp.plan_wave_prefix_sharing(prompts, 16, threshold=2, chunk_tokens=256)
    wp.validate_wave_prefix_plan(plan, prompts)
    assert plan.computed_tokens < plan.prompt_tokens
    # doc 0 is shared by 5 prompts for 3 blocks, then by 4 for 3 more: two chained segments
    seg_members = sorted(len(s.members) for s in plan.segments)
    assert seg_members == [4, 4, 4, 5]
    child = next(s for s in plan.segments if s.parent_id is not None)
    assert plan.segments[child.parent_id].token_end == child.token_start
    assert sum(1 for it in plan.items if it.kind == "tail") == len(prompts)
    assert len(plan.chunks) > 1 and all(plan.chunks)


def test_threshold_and_pool_budget():
    prompts = _wave(1)
    loose = wp.plan_wave_prefix_sharing(prompts, 16, threshold=2)
    strict = wp.plan_wave_prefix_sharing(prompts, 16, threshold=5)
    assert len(strict.segments) < len(loose.segments)
    small = wp.plan_wave_prefix_sharing(prompts, 16, threshold=2, pool_pages=3, chunk_tokens=10 ** 6)
    wp.validate_wave_prefix_plan(small, prompts)
    assert small.peak_pool_pages <= 3 or not small.segments


def test_materialized_prefix_kept_or_declined_by_name():
    block = 16
    base = list(range(block * 4))
    prompts = [base + [1, 2, 3], base + [4, 5], [9] * (block * 3) + [1]]
    # row 2 restores 2 blocks from a committed trajectory: no in-wave chain competes -> kept, saves all of it
    plan = wp.plan_wave_prefix_sharing(prompts, block, materialized=[wp.MaterializedPrefix(2, 2 * block)])
    wp.validate_wave_prefix_plan(plan, prompts)
    mat = [s for s in plan.segments if s.materialized]
    assert len(mat) == 1 and mat[0].members == (2,)
    assert any(it.kind == "materialize" for it in plan.items)
    # row 0 could restore 1 block, but the in-wave chain with row 1 is 4 blocks long: declined by name
    plan = wp.plan_wave_prefix_sharing(prompts, block, materialized=[wp.MaterializedPrefix(0, block)])
    assert plan.declined_materialized == {0: wp.DECLINED_POOL_CHAIN_LONGER}
    with pytest.raises(ValueError):
        wp.plan_wave_prefix_sharing(prompts, block, materialized=[wp.MaterializedPrefix(0, block + 1)])


def test_rank_packing_keeps_families_and_balances():
    prompts = _wave(2)
    pk = wp.pack_wave_ranks(prompts, 4, 16)
    assert len(pk.rank_of) == len(prompts) and set(pk.rank_of) <= set(range(4))
    assert pk.digest == wp.pack_wave_ranks(prompts, 4, 16).digest
    prof = wp.CostProfile(a=0.01, b=0.5, c=2.0, d=0.1, e=0.02)
    pk2 = wp.pack_wave_ranks(prompts, 2, 16, profile=prof)
    assert pk2.makespan > 0
    # one giant family on 2 ranks gets split when that lowers the makespan
    fam = [[5] * 32 + [i] * 8 for i in range(8)]
    pk3 = wp.pack_wave_ranks(fam, 2, 16)
    assert set(pk3.rank_of) == {0, 1}
    assert wp.find_cost_profile("m", "b200", 1) is None
    wp.register_cost_profile("m", "b200", 1, prof)
    assert wp.find_cost_profile("m", "b200", 1) is prof
    assert wp.first_divergence(["a", "a"], [[0, 1], [0, 1]]) is None
    assert wp.first_divergence(["a", "b"], [[0, 1, 1], [0, 0, 1]]) == 1

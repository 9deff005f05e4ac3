"""Tiny DeepSeek-V3-style MoE on CPU, fp32, world_size 1: engine == naive oracle, batch completes."""
import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.models.naive import NaiveModel
from batchgen_b200.models.transformer import AttnMeta
from batchgen_b200.models.weights import WeightSource
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range
from batchgen_b200.runtime.sequence import SamplingParams, SequenceStatus


def _prompts(cfg, n, length, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(2, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]


def _engine(cfg, pages=64, **kw):
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1,
                        decision_frequency_pages=1, **kw)
    return Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=pages)


def test_prefill_logits_match_naive():
    cfg = get_model_config("tiny-deepseek-v3")
    model = build_model(cfg, seed=0)
    naive = NaiveModel(cfg, WeightSource(seed=0))
    kv = PagedKVCache(cfg, 8, 16, "cpu", torch.float32)
    ids = _prompts(cfg, 1, 40)[0]
    pages = kv.alloc.alloc(3)
    meta = AttnMeta(mode="prefill", positions=torch.arange(40, dtype=torch.int32),
                    slot_mapping=torch.tensor(slots_for_range(pages, 0, 40, 16)),
                    block_table=build_block_table([pages], "cpu"), cu_seqlens=[0, 40], ctx_lens=[0])
    got = model.forward(torch.tensor(ids, dtype=torch.int32), meta, kv)
    want = naive.logits(ids)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()


def test_batch_of_8_matches_naive_tokens():
    cfg = get_model_config("tiny-deepseek-v3")
    eng = _engine(cfg)
    prompts = _prompts(cfg, 8, 32)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16, ignore_eos=True))
    assert all(len(o) == 16 for o in outs)
    assert all(s.status == SequenceStatus.COMPLETED for s in eng.seqs.values())
    assert eng.kv.alloc.num_used == 0
    naive = NaiveModel(cfg, WeightSource(seed=0))
    for p, o in list(zip(prompts, outs))[:3]:
        assert naive.generate(p, 16) == o


def test_small_pool_forces_waves_and_same_tokens():
    cfg = get_model_config("tiny-deepseek-v3")
    prompts = _prompts(cfg, 6, 32, seed=3)
    params = SamplingParams(max_new_tokens=24, ignore_eos=True)
    big = _engine(cfg, pages=128).generate(prompts, params)
    small_eng = _engine(cfg, pages=14)
    small = small_eng.generate(prompts, params)
    assert small == big
    assert small_eng.stats.prefill_waves > 1 or small_eng.stats.evictions > 0 or small_eng.stats.holds > 0


def test_prefix_cache_reuses_pages_and_keeps_tokens():
    cfg = get_model_config("tiny-deepseek-v3")
    shared = _prompts(cfg, 1, 48, seed=5)[0]
    prompts = [shared + tail for tail in _prompts(cfg, 4, 8, seed=6)]
    params = SamplingParams(max_new_tokens=8, ignore_eos=True)
    base = _engine(cfg, pages=128).generate(prompts, params)
    eng = _engine(cfg, pages=128, enable_prefix_cache=True)
    first = eng.generate(prompts[:1], params)
    rest = eng.generate(prompts[1:], params)
    assert first + rest == base
    assert eng.stats.prefill_cached_tokens >= 3 * 48
    assert eng.prefix.stats()["hits"] >= 3


def test_eos_stops_and_length_cap():
    cfg = get_model_config("tiny-deepseek-v3")
    eng = _engine(cfg)
    p = _prompts(cfg, 1, 20)[0]
    free_run = eng.generate([p], SamplingParams(max_new_tokens=12, ignore_eos=True))[0]
    cfg2 = get_model_config("tiny-deepseek-v3", eos_token_id=free_run[4])
    eng2 = Engine(build_model(cfg2, seed=0), eng.ecfg, num_gpu_pages=64)
    s = eng2.add_request(p, SamplingParams(max_new_tokens=12))
    eng2.run_to_completion()
    assert s.finish_reason == "stop" and s.output_ids == free_run[: free_run.index(free_run[4]) + 1]


def test_host_tier_hold_and_reload_same_tokens():
    cfg = get_model_config("tiny-deepseek-v3")
    prompts = _prompts(cfg, 5, 32, seed=9)
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    big = _engine(cfg, pages=256).generate(prompts, params)
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1,
                        decision_frequency_pages=1)
    eng = Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=18, num_host_pages=64)
    assert eng.generate(prompts, params) == big


def test_full_host_tier_evicts_parked_rows_by_growth_debt():
    """The host tier is too small for every parked row: parked rows with the least decoded give their pages up
    (and are re-prefilled later) only when another row must be parked; the tokens do not change."""
    cfg = get_model_config("tiny-deepseek-v3")
    prompts = _prompts(cfg, 8, 32, seed=9)
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    big = _engine(cfg, pages=256).generate(prompts, params)
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1,
                        decision_frequency_pages=1)
    eng = Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=14, num_host_pages=6)
    assert eng.generate(prompts, params) == big
    assert eng.stats.growth_evictions > 0 and eng.stats.evictions >= eng.stats.growth_evictions
    assert eng.chunk_sizer.completed_count == 8 and eng.chunk_sizer.ema_decode_length == 40.0


def test_chunked_prefill_of_long_prompts_matches_one_shot():
    """Prompts longer than max_prefill_tokens are computed in pieces; tokens equal the one-shot prefill, for the
    dense-attention model and for the DSA model (its indexer scores the keys written by earlier pieces)."""
    for name in ("tiny-deepseek-v3", "tiny-glm5"):
        cfg = get_model_config(name)
        prompts = _prompts(cfg, 3, 90, seed=21) + _prompts(cfg, 1, 17, seed=22)
        params = SamplingParams(max_new_tokens=5, ignore_eos=True)
        outs = []
        for cap in (8192, 32):
            for prefix in (False, True):
                ecfg = EngineConfig(page_size=16, max_prefill_tokens=cap, enable_prefix_cache=prefix)
                eng = Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=64)
                outs.append(eng.generate(prompts, params))
                assert (eng.stats.prefill_chunks > 0) == (cap == 32), (name, cap, prefix)
        assert all(o == outs[0] for o in outs[1:]), name


def test_other_families_run_and_match_naive():
    for name in ("tiny-glm5", "tiny-kimi-k3"):
        cfg = get_model_config(name)
        eng = _engine(cfg)
        prompts = _prompts(cfg, 2, 24, seed=11)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
        naive = NaiveModel(cfg, WeightSource(seed=0))
        assert naive.generate(prompts[0], 6) == outs[0], name


def test_legacy_and_gqa_families_match_naive():
    """GQA attention (sinks, sliding window, projection bias), Mixtral / DeepSeek-V2 / Qwen2-MoE routing and the gated
    shared expert: the engine's tokens equal the textbook model's."""
    for name in ("tiny-gpt-oss", "tiny-mixtral", "tiny-qwen2-moe", "tiny-deepseek-v2"):
        cfg = get_model_config(name)
        eng = _engine(cfg)
        prompts = _prompts(cfg, 2, 24, seed=13)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
        naive = NaiveModel(cfg, WeightSource(seed=0))
        assert naive.generate(prompts[1], 6) == outs[1], name


def test_router_scoring_modes():
    from batchgen_b200.ops import ref
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(5, 16, generator=g)
    idx, w = ref.router_topk(logits, None, 4, n_group=4, topk_group=2, norm_topk_prob=False, scale=2.0,
                             scoring="softmax_all")
    p = torch.softmax(logits, -1)
    for t in range(5):
        best = p[t].view(4, 4).max(-1)[0].topk(2)[1].tolist()
        allowed = [e for e in range(16) if e // 4 in best]
        want = sorted(allowed, key=lambda e: -float(p[t, e]))[:4]
        assert idx[t].tolist() == want
        assert torch.allclose(w[t], 2.0 * p[t, idx[t].long()])
    bias = torch.randn(16, generator=g) * 0.1
    idx, w = ref.router_topk(logits, bias, 3, scale=1.5, scoring="sqrtsoftplus")
    sc = torch.sqrt(torch.log1p(torch.exp(logits)))
    assert idx.tolist() == (sc + bias).topk(3)[1].tolist()
    sel = sc.gather(1, idx.long())
    assert torch.allclose(w, 1.5 * sel / sel.sum(-1, keepdim=True), atol=1e-6)

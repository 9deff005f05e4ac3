"""DeepSeek-V4 on CPU, fp32: window rings, pooled entries (plain and overlapped windows), indexer top-k,
hyper-connections and hash routing against the textbook model; chunked prefill and engine scheduling keep tokens."""
import pytest
import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.models.deepseek_v4 import CompressorWeights, pool_windows
from batchgen_b200.models.naive_v4 import NaiveV4
from batchgen_b200.models.transformer import AttnMeta
from batchgen_b200.models.weights import WeightSource
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range, v4_entries_per_page
from batchgen_b200.runtime.sequence import SamplingParams


def _ids(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist()


def _forward_chunks(model, kv, ids, cuts, pages, slot):
    """Prefill ``ids`` in chunks ending at ``cuts``; returns the logits of every position."""
    out, start = [], 0
    for end in cuts:
        n = end - start
        meta = AttnMeta(mode="prefill", positions=torch.arange(start, end, dtype=torch.int32),
                        slot_mapping=torch.tensor(slots_for_range(pages, start, end, kv.page_size)),
                        block_table=build_block_table([pages], "cpu"), cu_seqlens=[0, n], ctx_lens=[start],
                        state_slots=torch.tensor([slot], dtype=torch.int32))
        out.append(model.forward(torch.tensor(ids[start:end], dtype=torch.int32), meta, kv))
        start = end
    return torch.cat(out)


def test_prefill_logits_match_textbook_model():
    cfg = get_model_config("tiny-deepseek-v4")
    model = build_model(cfg, seed=0)
    kv = PagedKVCache(cfg, 8, 16, "cpu", torch.float32, state_slots=2)
    ids = _ids(cfg, 45)
    got = _forward_chunks(model, kv, ids, [45], kv.alloc.alloc(3), kv.state.acquire())
    want = NaiveV4(cfg, WeightSource(seed=0)).logits(ids)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), (got - want).abs().max()


@pytest.mark.parametrize("cuts", [[7, 20, 45], [1, 2, 3, 4, 5, 45], [16, 32, 44, 45]])
def test_chunked_prefill_and_single_token_steps_equal_one_pass(cuts):
    cfg = get_model_config("tiny-deepseek-v4")
    model = build_model(cfg, seed=0)
    ids = _ids(cfg, 45, seed=3)
    kv = PagedKVCache(cfg, 8, 16, "cpu", torch.float32, state_slots=2)
    whole = _forward_chunks(model, kv, ids, [45], kv.alloc.alloc(3), kv.state.acquire())
    kv2 = PagedKVCache(cfg, 8, 16, "cpu", torch.float32, state_slots=2)
    kv2.state.acquire()                                     # a different slot and different pages
    parts = _forward_chunks(model, kv2, ids, cuts, list(reversed(kv2.alloc.alloc(3))), kv2.state.acquire())
    assert torch.allclose(parts, whole, atol=1e-4, rtol=1e-3), (parts - whole).abs().max()


def test_pool_windows_state_carries_open_and_previous_window():
    torch.manual_seed(0)
    r, d, n = 4, 6, 19
    cw = CompressorWeights(ape=torch.randn(r, 2 * d), ratio=r, width=d)
    kv, sc = torch.randn(n, 2 * d), torch.randn(n, 2 * d)

    def run(cuts):
        pk, ps = torch.zeros(2 * r, 2 * d), torch.zeros(2 * r, 2 * d)
        ps[:r] = float("-inf")
        out, a = [], 0
        for b in cuts:
            out.append(pool_windows(kv[a:b], sc[a:b], a, cw, pk, ps))
            a = b
        return torch.cat(out)

    one = run([n])
    assert one.shape == (n // r, d)
    for cuts in ([3, 4, 5, 11, 19], list(range(1, n + 1))):
        assert torch.allclose(run(cuts), one, atol=1e-6)
    # entry 1 by hand: previous window through the lower half, own window through the upper half
    rows = torch.cat([kv[0:4, :d], kv[4:8, d:]])
    gate = torch.cat([(sc[0:4] + cw.ape)[:, :d], (sc[4:8] + cw.ape)[:, d:]])
    assert torch.allclose(one[1], (rows * torch.softmax(gate, 0)).sum(0), atol=1e-6)


def test_entries_per_page_rule():
    assert v4_entries_per_page(4, 64) == 16 and v4_entries_per_page(128, 64) == 1 and v4_entries_per_page(64, 64) == 1
    with pytest.raises(AssertionError):
        v4_entries_per_page(48, 64)


def _engine(cfg, pages=64, **kw):
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1,
                        decision_frequency_pages=1, **kw)
    return Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=pages)


def test_engine_tokens_match_textbook_model():
    cfg = get_model_config("tiny-deepseek-v4")
    eng = _engine(cfg)
    prompts = [_ids(cfg, n, seed=10 + n) for n in (40, 23, 9)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    naive = NaiveV4(cfg, WeightSource(seed=0))
    assert naive.generate(prompts[1], 12) == outs[1]
    assert naive.generate(prompts[2], 12) == outs[2]
    assert eng.kv.alloc.num_used == 0 and eng.kv.state.num_free == eng.kv.state.num_slots


def test_engine_small_pool_chunked_prefill_and_host_tier_keep_tokens():
    cfg = get_model_config("tiny-deepseek-v4")
    prompts = [_ids(cfg, 32, seed=20 + i) for i in range(6)]
    params = SamplingParams(max_new_tokens=24, ignore_eos=True)
    big = _engine(cfg, pages=128).generate(prompts, params)
    small = _engine(cfg, pages=14)
    assert small.generate(prompts, params) == big
    assert small.stats.prefill_waves > 1 or small.stats.evictions > 0 or small.stats.holds > 0
    chunked = _engine(cfg, pages=128, max_prefill_tokens=24)
    assert chunked.generate(prompts, params) == big
    assert chunked.stats.prefill_chunks > 0


def test_parked_sequences_move_window_and_compressor_state_to_host_and_back():
    cfg = get_model_config("tiny-deepseek-v4")
    prompts = [_ids(cfg, 32, seed=30 + i) for i in range(5)]
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    want = _engine(cfg, pages=256, max_decode_batch=8).generate(prompts, params)
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1,
                        max_decode_batch=8, max_state_slots=5)
    eng = Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=18, num_host_pages=64)
    assert eng.generate(prompts, params) == want
    assert eng.stats.holds > 0 and eng.host_state.offloads > 0 and eng.host_state.loads == eng.host_state.offloads
    assert eng.kv.state.num_free == 5 and eng.host_state.num_free == eng.host_state.num_items


def test_prefix_cache_is_refused():
    cfg = get_model_config("tiny-deepseek-v4")
    with pytest.raises(ValueError):
        _engine(cfg, enable_prefix_cache=True)


def test_full_size_presets_describe_the_published_models():
    flash, pro = get_model_config("deepseek-v4-flash"), get_model_config("DeepSeek-V4-Pro")
    assert len(flash.compress_ratios) == flash.num_layers == 43 and flash.compress_ratios[:4] == (0, 0, 4, 128)
    assert len(pro.compress_ratios) == pro.num_layers == 61 and pro.compress_ratios[:3] == (128, 128, 4)
    assert 2.7e11 < flash.param_count() < 3.0e11 and 1.5e12 < pro.param_count() < 1.7e12
    assert flash.kv_bytes_per_token() < 8000                 # pooled entries only: a tenth of a DeepSeek-V3 row


def test_batched_decode_equals_row_by_row_decode():
    """The decode step that handles all rows at once (no host reads: open windows write a scratch entry, closing
    windows overwrite it) gives the tokens of the row-by-row routine that the prefill chunks use."""
    cfg = get_model_config("tiny-deepseek-v4")
    prompts = [_ids(cfg, n, seed=40 + n) for n in (5, 17, 30, 3)]
    params = SamplingParams(max_new_tokens=20, ignore_eos=True)
    outs = []
    for batched in (True, False):
        eng = _engine(cfg)
        eng.model.batched_decode = batched
        outs.append(eng.generate(prompts, params))
    assert outs[0] == outs[1]


def test_decode_rows_without_a_sequence_touch_nothing():
    cfg = get_model_config("tiny-deepseek-v4")
    model = build_model(cfg, seed=0)

    def run(pad):
        kv = PagedKVCache(cfg, 8, 16, "cpu", torch.float32, state_slots=3)
        pages = [kv.alloc.alloc(2), kv.alloc.alloc(2)]
        slots = [kv.state.acquire(), kv.state.acquire()]
        lens = [15, 7]                                          # the first row's next token closes windows of 4 and 8
        for i, n in enumerate(lens):
            _forward_chunks(model, kv, _ids(cfg, n, seed=50 + i), [n], pages[i], slots[i])
        rows = [(0, 11), (1, 13)] + ([(-1, 0)] * pad)
        bt = build_block_table([pages[i] if i >= 0 else [0, 0] for i, _ in rows], "cpu")
        meta = AttnMeta(mode="decode", positions=torch.tensor([lens[i] if i >= 0 else 0 for i, _ in rows], dtype=torch.int32),
                        slot_mapping=torch.tensor([slots_for_range(pages[i], lens[i], lens[i] + 1, 16)[0] if i >= 0 else -1
                                                   for i, _ in rows]),
                        block_table=bt, seqlens=torch.tensor([lens[i] + 1 if i >= 0 else 1 for i, _ in rows], dtype=torch.int32),
                        state_slots=torch.tensor([slots[i] if i >= 0 else -1 for i, _ in rows], dtype=torch.int32))
        out = model.forward(torch.tensor([t for _, t in rows], dtype=torch.int32), meta, kv)
        return out[:2], kv.v4_comp[1][: kv.num_pages].clone(), kv.state.rec[0, :3].clone()

    a, b = run(0), run(2)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-6)


def test_decode_core_through_the_mla_decode_routine_matches_the_plain_softmax():
    """The decode core expressed for the absorbed-MLA decode kernel (sink as an appended row scored through a flag
    column, masked rows pushed out through a second flag column) gives the tokens of the plain masked softmax."""
    cfg = get_model_config("tiny-deepseek-v4")
    prompts = [_ids(cfg, n, seed=60 + n) for n in (5, 17, 30, 3)]
    params = SamplingParams(max_new_tokens=20, ignore_eos=True)
    outs = []
    for route in (False, True):
        eng = _engine(cfg)
        eng.model.kernel_math_anywhere = route
        outs.append(eng.generate(prompts, params))
    assert outs[0] == outs[1]


def test_ratio_larger_than_the_page_places_one_entry_every_few_pages():
    """Compression ratio 32 with 16-token pages: entry c sits in page 2c of the sequence (slot 0); whole-prompt, chunked
    and decode paths agree with the textbook model."""
    cfg = get_model_config("tiny-deepseek-v4", compress_ratios=(32, 4), num_layers=2, num_hash_layers=0)
    model = build_model(cfg, seed=0)
    ids = _ids(cfg, 100, seed=70)
    want = NaiveV4(cfg, WeightSource(seed=0)).logits(ids)
    kv = PagedKVCache(cfg, 16, 16, "cpu", torch.float32, state_slots=2)
    got = _forward_chunks(model, kv, ids, [100], kv.alloc.alloc(7), kv.state.acquire())
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), (got - want).abs().max()
    kv2 = PagedKVCache(cfg, 16, 16, "cpu", torch.float32, state_slots=2)
    parts = _forward_chunks(model, kv2, ids, [31, 32, 33, 64, 95, 96, 100], list(reversed(kv2.alloc.alloc(7))), kv2.state.acquire())
    assert torch.allclose(parts, want, atol=1e-4, rtol=1e-3), (parts - want).abs().max()
    eng = _engine(cfg)
    prompt = ids[:60]
    got_tokens = eng.generate([prompt], SamplingParams(max_new_tokens=10, ignore_eos=True))[0]
    assert got_tokens == NaiveV4(cfg, WeightSource(seed=0)).generate(prompt, 10)

"""Host KV tier on the native engine (node-shared region + asynchronous movers) under the real scheduler."""
import pytest
import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.sequence import SamplingParams

pytestmark = pytest.mark.gpu


def _cfg():
    return get_model_config("tiny-deepseek-v3", hidden_size=1024, q_lora_rank=512, kv_lora_rank=512,
                            qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_heads=16,
                            intermediate_size=2048, moe_intermediate_size=512, n_routed_experts=16,
                            num_experts_per_tok=4, n_group=4, topk_group=2, vocab_size=4096, quant="fp8_block")


def _prompts(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def test_oversubscribed_device_pool_parks_rows_in_the_native_tier():
    """Eight rows need about 3x the device pool: rows are parked in the host region and brought back, with the same
    schedule and tokens as the pinned-tensor tier, and the first tokens of an engine that never parks anything."""
    from batchgen_b200.ops import _ext
    cfg = _cfg()
    prompts = _prompts(cfg, (100, 150, 70, 130, 90, 160, 110, 140), seed=3)
    params = SamplingParams(max_new_tokens=120, ignore_eos=True)
    roomy = Engine(build_model(cfg, "cuda", "bf16", seed=0), EngineConfig(page_size=64), num_gpu_pages=256)
    want = roomy.generate(prompts, params)
    outs, engines = [], []
    for backend in ("torch", "native"):
        ecfg = EngineConfig(page_size=64, initial_gpu_page_buffer=1, extension_gpu_page_buffer=1,
                            decision_frequency_pages=1, host_kv_backend=backend)
        eng = Engine(build_model(cfg, "cuda", "bf16", seed=0), ecfg, num_gpu_pages=12, num_host_pages=64)
        outs.append(eng.generate(prompts, params))
        torch.cuda.synchronize()
        _ext.check_status()
        engines.append(eng)
    native = engines[1]
    assert native.host_tier is not None and engines[0].host_tier is None
    assert native.stats.holds > 0 and native.stats.loads > 0
    assert native.stats.holds == engines[0].stats.holds              # same schedule
    assert outs[1] == outs[0]
    assert [o[0] for o in outs[1]] == [o[0] for o in want]
    assert all(len(o) == 120 for o in outs[1])
    st = native.host_tier.stats()
    assert st["offloaded_pages"] > 0 and st["loaded_pages"] > 0 and st["bytes_moved"] > 0
    native._drain_deferred(block=True)
    assert native.host_tier.region.audit() == 0
    assert native.host_tier.region.num_free == native.host_tier.region.num_pages
    assert native.kv.alloc.num_free == 12
    native.host_tier.close()


def test_prefix_pages_demoted_to_host_come_back():
    """A finished turn's pages leave the device cache under pressure, stay in the host coordinator, and are promoted
    when the next turn of the conversation arrives."""
    cfg = _cfg()
    first = _prompts(cfg, (400,), seed=5)[0]                     # 6 full pages
    others = _prompts(cfg, (300, 310, 320), seed=6)
    params = SamplingParams(max_new_tokens=8, ignore_eos=True)
    ecfg = EngineConfig(page_size=64, enable_prefix_cache=True)
    eng = Engine(build_model(cfg, "cuda", "bf16", seed=0), ecfg, num_gpu_pages=16, num_host_pages=64)
    out1 = eng.generate([first], params)[0]
    assert len(eng.prefix) == 6                                   # the turn's six full pages stay cached
    eng.generate(others, params)                                  # 3 x 6 pages: the cached turn must yield
    assert eng.host_tier.demoted_pages > 0
    turn2 = first + out1 + _prompts(cfg, (50,), seed=7)[0]
    got = eng.generate([turn2], params)[0]
    assert eng.stats.prefix_promoted_pages > 0
    fresh = Engine(build_model(cfg, "cuda", "bf16", seed=0), EngineConfig(page_size=64), num_gpu_pages=64)
    assert fresh.generate([turn2], params)[0][:2] == got[:2]
    eng.host_tier.close()

"""KDA (gated delta-rule linear attention): op-level reference properties and the engine on a model with
KDA layers against the naive oracle (CPU, fp32)."""
import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.models.naive import NaiveModel
from batchgen_b200.models.weights import WeightSource
from batchgen_b200.ops import kda
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.sequence import SamplingParams


def _inputs(T, H, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    HD = H * D
    qkv = torch.randn(T, 3 * HD, generator=g)
    f = torch.randn(T, HD, generator=g)
    beta = torch.randn(T, H, generator=g)
    z = torch.randn(T, HD, generator=g)
    p = kda.KDAParams(conv_w=torch.randn(3 * HD, 4, generator=g) * 0.5, conv_b=None,
                      A_log=torch.randn(H, generator=g) * 0.3, dt_bias=torch.randn(HD, generator=g) * 0.3,
                      norm_w=1.0 + 0.1 * torch.randn(D, generator=g))
    return qkv, f, beta, z, p


def test_chunked_prefill_and_decode_continue_the_same_state():
    H, D, T = 2, 16, 11
    qkv, f, beta, z, p = _inputs(T, H, D)
    conv = torch.zeros(3, 3 * H * D, 3)
    rec = torch.zeros(3, H, D, D)
    whole = kda.kda_forward(qkv, f, beta, z, p, conv, rec, [1], [0, T], [0], H, D, D ** -0.5, 1e-6)
    # the same tokens as a 6-token chunk, a 4-token continuation and one decode step, in another slot
    a = kda.kda_forward(qkv[:6], f[:6], beta[:6], z[:6], p, conv, rec, [2], [0, 6], [0], H, D, D ** -0.5, 1e-6)
    b = kda.kda_forward(qkv[6:10], f[6:10], beta[6:10], z[6:10], p, conv, rec, [2], [0, 4], [1], H, D, D ** -0.5, 1e-6)
    c = kda.kda_forward(qkv[10:], f[10:], beta[10:], z[10:], p, conv, rec, [2], None, None, H, D, D ** -0.5, 1e-6)
    assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-5, rtol=1e-5)
    assert torch.allclose(rec[1], rec[2], atol=1e-6) and torch.allclose(conv[1], conv[2])
    assert rec[0].abs().max() == 0                       # untouched slot


def test_packed_sequences_are_independent_and_negative_slots_are_skipped():
    H, D = 2, 16
    qkv, f, beta, z, p = _inputs(9, H, D, seed=1)
    conv = torch.zeros(4, 3 * H * D, 3)
    rec = torch.zeros(4, H, D, D)
    out = kda.kda_forward(qkv, f, beta, z, p, conv, rec, [0, -1, 3], [0, 4, 6, 9], [0, 0, 0], H, D, 0.25, 1e-6)
    conv2, rec2 = torch.zeros_like(conv), torch.zeros_like(rec)
    solo = kda.kda_forward(qkv[6:], f[6:], beta[6:], z[6:], p, conv2, rec2, [1], [0, 3], [0], H, D, 0.25, 1e-6)
    assert torch.allclose(out[6:], solo, atol=1e-6)
    assert out[4:6].abs().max() == 0 and rec[1].abs().max() == 0
    assert torch.allclose(rec[3], rec2[1])


def test_decay_bounds_and_delta_rule_fixed_point():
    H, D = 1, 8
    g = kda.kda_gate(torch.randn(5, H * D), torch.zeros(H), torch.zeros(H * D), H, D)
    assert (g <= 0).all()
    # with no decay and beta = 1, writing (k, v) then reading with q = k returns v exactly (k has unit norm)
    k = torch.randn(1, H, D)
    v = torch.randn(1, H, D)
    S = torch.zeros(H, D, D)
    o = kda.kda_recurrent_ref(k.clone(), k.clone(), v, torch.zeros(1, H, D), torch.ones(1, H), S, 1.0)
    assert torch.allclose(o, v, atol=1e-4)


def test_engine_with_kda_layers_matches_naive_oracle():
    cfg = get_model_config("tiny-kimi-linear")
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=11)
    ecfg = EngineConfig(page_size=16, max_decode_batch=4, max_state_slots=2, enable_cuda_graph=False)
    eng = Engine(model, ecfg, num_gpu_pages=64)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 17, 5)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True))
    oracle = NaiveModel(cfg, WeightSource(seed=11))
    for pr, o in zip(prompts, outs):
        assert o == oracle.generate(pr, 4)
    assert eng.kv.state.num_free == 2                    # three sequences shared two slots and returned them
    assert eng.kv.kv.shape[0] == 1                       # only the MLA layer owns paged KV


def test_parked_sequences_move_their_state_to_host_and_back():
    """Few GPU pages and a host tier: rows are put on hold and resumed; the recurrent state of a held row travels
    to the host store and returns to whatever slot is free, and the tokens equal an unconstrained run."""
    cfg = get_model_config("tiny-kimi-linear")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(2, cfg.vocab_size, (32,), generator=g).tolist() for _ in range(5)]
    params = SamplingParams(max_new_tokens=40, temperature=0.0, ignore_eos=True)
    big = Engine(build_model(cfg, device="cpu", dtype=torch.float32, seed=0),
                 EngineConfig(page_size=16, max_decode_batch=8, enable_cuda_graph=False), num_gpu_pages=256)
    want = big.generate(prompts, params)
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1,
                        max_decode_batch=8, max_state_slots=5, enable_cuda_graph=False)
    eng = Engine(build_model(cfg, device="cpu", dtype=torch.float32, seed=0), ecfg, num_gpu_pages=18, num_host_pages=64)
    assert eng.host_state is not None
    assert eng.generate(prompts, params) == want
    assert eng.stats.holds > 0 and eng.host_state.offloads > 0 and eng.host_state.loads == eng.host_state.offloads
    assert eng.kv.state.num_free == 5 and eng.host_state.num_free == eng.host_state.num_items


def test_kda_layers_with_a_dsa_indexed_mla_layer_match_naive():
    cfg = get_model_config("tiny-kimi-k3.1")
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=5)
    eng = Engine(model, EngineConfig(page_size=16, max_decode_batch=4, enable_cuda_graph=False), num_gpu_pages=64)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 21)]   # longer than top-k 16
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True))
    oracle = NaiveModel(cfg, WeightSource(seed=5))
    for pr, o in zip(prompts, outs):
        assert o == oracle.generate(pr, 4)
    assert get_model_config("kimi-k3.1").has_dsa and len(get_model_config("kimi-k3.1").indexer_full_layers) == 24


def test_chunk_form_equals_the_recurrence():
    g0 = torch.Generator().manual_seed(4)
    n, H, D = 150, 2, 16
    q, k, v = (torch.randn(n, H, D, generator=g0) for _ in range(3))
    g = -torch.rand(n, H, D, generator=g0) * 0.3
    beta = torch.rand(n, H, generator=g0)
    S0 = torch.randn(H, D, D, generator=g0) * 0.2
    Sa, Sb = S0.clone(), S0.clone()
    a = kda.kda_recurrent_ref(q, k, v, g, beta, Sa, 0.25)
    b = kda.kda_chunk_ref(q, k, v, g, beta, Sb, 0.25, chunk=64)
    assert torch.allclose(a, b, atol=2e-4, rtol=2e-4)
    assert torch.allclose(Sa, Sb, atol=2e-4, rtol=2e-4)


def test_chunked_prefill_advances_the_recurrent_state_in_every_piece():
    """A prompt cut into pieces by ``max_prefill_tokens``: every piece (not only the last, which samples) updates the
    sequence's state slot, so the tokens equal the one-pass run."""
    cfg = get_model_config("tiny-kimi-linear")
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(2, cfg.vocab_size, (40,), generator=g).tolist() for _ in range(3)]
    params = SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True)
    mk = lambda **kw: Engine(build_model(cfg, device="cpu", dtype=torch.float32, seed=0),
                             EngineConfig(page_size=16, max_decode_batch=8, enable_cuda_graph=False, **kw), num_gpu_pages=64)
    want = mk().generate(prompts, params)
    eng = mk(max_prefill_tokens=24)
    assert eng.generate(prompts, params) == want
    assert eng.stats.prefill_chunks > 0

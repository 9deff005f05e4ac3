"""KDA kernel (conv + gated delta rule + gated norm, prefill and decode) against the fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _inputs(T, H, D, seed=0):
    from batchgen_b200.ops import kda
    g = torch.Generator().manual_seed(seed)
    HD = H * D
    wide = torch.randn(T, 4 * HD + 24, generator=g).to(torch.bfloat16)     # q | k | v | z | beta (+ padding) in one buffer
    f = torch.randn(T, HD, generator=g).to(torch.bfloat16)
    p = kda.KDAParams(conv_w=torch.randn(3 * HD, 4, generator=g) * 0.5, conv_b=torch.randn(3 * HD, generator=g) * 0.1,
                      A_log=torch.randn(H, generator=g) * 0.3, dt_bias=torch.randn(HD, generator=g) * 0.3,
                      norm_w=1.0 + 0.1 * torch.randn(D, generator=g))
    return wide, f, p


def _views(wide, H, D):
    HD = H * D
    return wide[:, : 3 * HD], wide[:, 4 * HD: 4 * HD + H], wide[:, 3 * HD: 4 * HD]


@pytest.mark.parametrize("D,H", [(128, 3), (64, 4)])
def test_kda_prefill_continuation_and_decode(D, H):
    from batchgen_b200.ops import kda
    lens = [37, 1, 130]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    wide, f, p = _inputs(T, H, D)
    slots = [2, 0, 3]
    nslots = 5
    conv_c, rec_c = torch.zeros(nslots, 3 * H * D, 3), torch.zeros(nslots, H, D, D)
    g = torch.Generator().manual_seed(5)
    rec_c[3] = torch.randn(H, D, D, generator=g) * 0.1        # sequence 2 continues from a stored state
    conv_c[3] = torch.randn(3 * H * D, 3, generator=g)
    conv_g, rec_g = conv_c.cuda(), rec_c.cuda()
    qkv, beta, z = _views(wide.float(), H, D)
    want = kda.kda_forward(qkv, f.float(), beta, z, p, conv_c, rec_c, slots, cu, [0, 0, 1], H, D, D ** -0.5, 1e-6)
    pg = kda.KDAParams(*(None if t is None else t.cuda() for t in (p.conv_w, p.conv_b, p.A_log, p.dt_bias, p.norm_w)))
    wg = wide.cuda()
    qkv_g, beta_g, z_g = _views(wg, H, D)
    got = kda.kda_forward(qkv_g, f.cuda(), beta_g, z_g, pg, conv_g, rec_g, slots, cu, [0, 0, 1], H, D, D ** -0.5, 1e-6)
    torch.cuda.synchronize()
    for i in range(3):
        assert _rel(got[cu[i]:cu[i + 1]].cpu(), want[cu[i]:cu[i + 1]]) < 2e-2, i
    assert _rel(rec_g.cpu(), rec_c) < 1e-3 and _rel(conv_g.cpu(), conv_c) < 1e-6
    assert rec_g[1].abs().max() == 0 and rec_g[4].abs().max() == 0
    # one decode step for the three sequences plus a padding row (slot -1)
    wide2, f2, _ = _inputs(4, H, D, seed=9)
    qkv2, beta2, z2 = _views(wide2.float(), H, D)
    want2 = kda.kda_forward(qkv2, f2.float(), beta2, z2, p, conv_c, rec_c, slots + [-1], None, None, H, D, D ** -0.5, 1e-6)
    w2g = wide2.cuda()
    q2g, b2g, z2g = _views(w2g, H, D)
    got2 = kda.kda_forward(q2g, f2.cuda(), b2g, z2g, pg, conv_g, rec_g,
                           torch.tensor(slots + [-1], dtype=torch.int32, device="cuda"), None, None, H, D, D ** -0.5, 1e-6)
    torch.cuda.synchronize()
    assert _rel(got2[:3].cpu(), want2[:3]) < 2e-2
    assert _rel(rec_g.cpu(), rec_c) < 1e-3


def test_model_with_kda_layers_on_gpu_matches_cpu():
    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.sequence import SamplingParams
    from batchgen_b200.ops.policy import set_library_fallback
    cfg = get_model_config("tiny-kimi-linear")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 9)]
    logits = {}
    set_library_fallback(True)        # the MLA layer of this preset has a test-sized latent (64): library path
    for dev, dt in (("cpu", torch.float32), ("cuda", torch.bfloat16)):
        model = build_model(cfg, device=dev, dtype=dt, seed=4)
        eng = Engine(model, EngineConfig(page_size=64, max_decode_batch=4, enable_cuda_graph=False, device=dev),
                     num_gpu_pages=16)
        seen = []
        orig = model.forward

        def spy(ids, meta, cache, _o=orig, _s=seen):
            out = _o(ids, meta, cache)
            _s.append(out.float().cpu())
            return out
        model.forward = spy
        eng.generate(prompts, SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True))
        logits[dev] = seen
    set_library_fallback(False)
    # prefill logits and the first decode step (same tokens fed as long as greedy picks agree; compare what is comparable)
    assert _rel(logits["cuda"][0], logits["cpu"][0]) < 0.06

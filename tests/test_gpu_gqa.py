"""Paged GQA decode kernel (sinks, sliding window, split KV) against the fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Hq,Hkv,D", [(64, 8, 64), (48, 8, 128), (8, 8, 64)])
@pytest.mark.parametrize("window,use_sinks,splits", [(0, False, 1), (128, True, 1), (0, True, 3), (100, False, 2)])
def test_gqa_decode(Hq, Hkv, D, window, use_sinks, splits):
    from batchgen_b200.ops import _ext, attention, ref
    g = torch.Generator().manual_seed(Hq + D + window)
    page, lens = 64, [1, 63, 64, 65, 300, 517]
    B = len(lens)
    npg = [(n + page - 1) // page for n in lens]
    cache = (torch.randn(sum(npg) + 2, page, 2 * Hkv * D, generator=g) * 0.7).to(torch.bfloat16)
    bt = torch.zeros(B, max(npg), dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(npg):
        bt[b, :n] = torch.arange(nxt, nxt + n)
        nxt += n
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
    sinks = torch.randn(Hq, generator=g) if use_sinks else None
    sl = torch.tensor(lens, dtype=torch.int32)
    scale = D ** -0.5
    got = attention.gqa_decode(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), Hkv, scale, window=window,
                               sinks=sinks.cuda() if use_sinks else None, num_splits=splits).cpu().float()
    _ext.check_status()
    want = attention.gqa_decode(q.float(), cache.float(), bt, sl, Hkv, scale, window=window, sinks=sinks)
    err = ((got - want).norm() / want.norm()).item()
    assert err < 1.5e-2, err

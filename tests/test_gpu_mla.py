"""tcgen05 paged-MLA kernel (decode, split-KV, causal prefill) against the fp32 reference."""
import pytest
import torch

from batchgen_b200.ops import mla_cuda, ref
from batchgen_b200.ops.mla_kernel import mla_decode_tc, mla_prefill_tc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(B, H, lens, seed=0, pages_extra=3):
    g = torch.Generator(device=DEV).manual_seed(seed)
    S = 64
    need = [(l + S - 1) // S for l in lens]
    P = sum(need) + pages_extra
    cache = (torch.randn(P, S, 576, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(P, device=DEV, generator=g).to(torch.int32)
    bt = torch.zeros(B, max(need) + 1, dtype=torch.int32, device=DEV)
    o = 0
    for i, n in enumerate(need):
        bt[i, :n] = perm[o:o + n]
        o += n
    return cache, bt


def _check(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    scale = want.float().abs().max().item()
    assert err <= tol * scale, (err, scale)


@pytest.fixture(autouse=True)
def _status():
    from batchgen_b200.ops import _ext
    yield
    torch.cuda.synchronize()
    _ext.check_status()


@pytest.mark.parametrize("H", [16, 32, 128, 8])
@pytest.mark.parametrize("lens", [[1], [64, 65, 127, 128, 129], [700, 3, 2049, 300]])
def test_decode_matches_reference(H, lens):
    B = len(lens)
    cache, bt = _setup(B, H, lens)
    q = torch.randn(B, H, 576, device=DEV).to(torch.bfloat16)
    q_abs, q_pe = q[..., :512].contiguous(), q[..., 512:]
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 0.1
    got = mla_decode_tc(q_abs, q_pe, cache, bt, sl, scale, 512, num_splits=1)
    want = ref.mla_decode(q_abs.float().cpu(), q_pe.float().cpu(), cache.float().cpu(), bt.cpu(), sl.cpu(), scale, 512)
    _check(got.cpu(), want)


@pytest.mark.parametrize("splits", [2, 5])
def test_decode_split_kv(splits):
    lens = [1000, 130, 64, 2500]
    B, H = len(lens), 16
    cache, bt = _setup(B, H, lens, seed=1)
    q = torch.randn(B, H, 576, device=DEV).to(torch.bfloat16)
    q_abs, q_pe = q[..., :512].contiguous(), q[..., 512:].contiguous()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = mla_decode_tc(q_abs, q_pe, cache, bt, sl, 0.07, 512, num_splits=splits)
    want = ref.mla_decode(q_abs.float().cpu(), q_pe.float().cpu(), cache.float().cpu(), bt.cpu(), sl.cpu(), 0.07, 512)
    _check(got.cpu(), want)


def test_decode_strided_qpe_and_large_scores():
    lens = [333, 900]
    B, H = 2, 16
    cache, bt = _setup(B, H, lens, seed=2)
    qfull = (torch.randn(B, H, 192, device=DEV) * 4).to(torch.bfloat16)     # large logits: exercises rescaling
    q_abs = (torch.randn(B, H, 512, device=DEV) * 2).to(torch.bfloat16)
    q_pe = qfull[..., 128:]
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = mla_decode_tc(q_abs, q_pe, cache, bt, sl, 0.3, 512, num_splits=1)
    want = ref.mla_decode(q_abs.float().cpu(), q_pe.float().cpu(), cache.float().cpu(), bt.cpu(), sl.cpu(), 0.3, 512)
    _check(got.cpu(), want, 3e-2)


@pytest.mark.parametrize("H", [16, 32, 8])
def test_prefill_causal_with_context(H):
    new = [70, 1, 200, 129]
    ctx = [0, 64, 100, 0]
    lens = [a + b for a, b in zip(new, ctx)]
    cache, bt = _setup(len(new), H, lens, seed=3)
    T = sum(new)
    q = torch.randn(T, H, 576, device=DEV).to(torch.bfloat16)
    q_abs, q_pe = q[..., :512].contiguous(), q[..., 512:]
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    got = mla_prefill_tc(q_abs, q_pe, cache, bt, cu, ctx, 0.1, 512)
    want = ref.mla_prefill(q_abs.float().cpu(), q_pe.float().cpu(), cache.float().cpu(), bt.cpu(), cu, ctx, 0.1, 512)
    _check(got.cpu(), want)


def test_library_path_agrees():
    lens = [500, 77]
    cache, bt = _setup(2, 16, lens, seed=4)
    q = torch.randn(2, 16, 576, device=DEV).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    a = mla_cuda.mla_decode_lib(q[..., :512].contiguous(), q[..., 512:].contiguous(), cache, bt, sl, 0.1, 512)
    b = mla_decode_tc(q[..., :512].contiguous(), q[..., 512:].contiguous(), cache, bt, sl, 0.1, 512)
    _check(b, a)


# ---------------------------------------------------------------- persistent decode kernel (heads % 64 == 0)
@pytest.mark.parametrize("H", [64, 128])
@pytest.mark.parametrize("lens", [[1], [64, 65, 127, 128, 129], [700, 3, 2049, 300], [0, 300, 0, 1]])
def test_persistent_decode_matches_reference(H, lens):
    from batchgen_b200.ops.mla_kernel import mla_decode_persist
    B = len(lens)
    cache, bt = _setup(B, H, lens, seed=5)
    q = torch.randn(B, H, 576, device=DEV).to(torch.bfloat16)
    q_abs, q_pe = q[..., :512], q[..., 512:]                      # strided views of one [B, H, 576] buffer
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for _ in range(2):                                            # twice: the pair counters must be back at zero
        got = mla_decode_persist(q_abs, q_pe, cache, bt, sl, 0.1)
        torch.cuda.synchronize()
    want = ref.mla_decode(q_abs.float().cpu(), q_pe.float().cpu(), cache.float().cpu(), bt.cpu(), sl.cpu(), 0.1, 512)
    live = [i for i, n in enumerate(lens) if n > 0]
    _check(got.cpu()[live], want[live])
    dead = [i for i, n in enumerate(lens) if n == 0]
    if dead:
        assert float(got[dead].float().abs().max()) == 0.0       # rows without tokens come out as zeros


@pytest.mark.parametrize("B,H,max_len,seed", [(200, 128, 3000, 7), (1, 128, 20000, 8), (48, 128, 2816, 9),
                                               (300, 64, 700, 10)])
def test_persistent_decode_cuts_and_merges(B, H, max_len, seed):
    """Ragged batches whose tile sequence is cut across CTAs inside pairs (partials + merge by the last arriver), one
    very long sequence cut across every CTA, and many short pairs per CTA; against the per-CTA kernel."""
    from batchgen_b200.ops.mla_kernel import mla_decode_persist
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(max(1, max_len // 8), max_len + 1, (B,), generator=g).tolist() if B > 1 else [max_len]
    cache, bt = _setup(B, H, lens, seed=seed)
    q = (torch.randn(B, H, 576, device=DEV) * 1.5).to(torch.bfloat16)
    q_abs, q_pe = q[..., :512].contiguous(), q[..., 512:].contiguous()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = mla_decode_persist(q_abs, q_pe, cache, bt, sl, 0.12)
    got2 = mla_decode_persist(q_abs, q_pe, cache, bt, sl, 0.12)
    want = mla_decode_tc(q_abs, q_pe, cache, bt, sl, 0.12, 512, num_splits=1)
    torch.cuda.synchronize()
    _check(got, want)
    assert torch.equal(got, got2)

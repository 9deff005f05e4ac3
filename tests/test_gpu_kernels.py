"""Each sm_100a kernel against the plain-PyTorch fp32 reference of the same operator."""
import pytest
import torch

from batchgen_b200.ops import fused, gemm, moe, ref, sampling

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def _close(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    scale = max(want.float().abs().max().item(), 1e-6)
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


@pytest.fixture(autouse=True)
def _status():
    from batchgen_b200.ops import _ext
    yield
    torch.cuda.synchronize()
    _ext.check_status()


@pytest.mark.parametrize("T,K", [(1, 128), (77, 1024), (300, 7168)])
@pytest.mark.parametrize("pow2", [False, True])
def test_act_quant_bytes_equal_reference(T, K, pow2):
    x = (torch.randn(T, K, device=DEV) * 3).to(torch.bfloat16)
    q, s = fused.act_quant(x, pow2_scale=pow2)
    qr, sr = ref.act_quant(x, 128, pow2)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    mism = (q.view(torch.uint8) != qr.view(torch.uint8)).float().mean().item()
    assert mism < 2e-3, mism          # rounding of x * (1/s) may differ by one ulp on a few elements
    _close(ref.dequant_act(q, s.contiguous()), ref.dequant_act(qr, sr), 7e-2)


def test_act_quant_silu_mul():
    x = torch.randn(50, 2 * 512, device=DEV, dtype=torch.bfloat16)
    q, s = fused.act_quant(x, silu_mul=True)
    qr, sr = ref.act_quant(ref.silu_mul(x))
    _close(ref.dequant_act(q, s.contiguous()), ref.dequant_act(qr, sr), 7e-2)


@pytest.mark.parametrize("H", [512, 6144, 7168])
def test_rmsnorm_variants(H):
    T = 37
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    y, _, _ = fused.rmsnorm(x, w, 1e-6)
    _close(y, ref.rmsnorm(x.float(), w.float(), 1e-6), 1e-2)
    r2 = r.clone()
    y2, q2, s2 = fused.rmsnorm(x, w, 1e-6, residual=r2, quant=True)
    want_r = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(r2, want_r)
    want_y = ref.rmsnorm(want_r.float(), w.float(), 1e-6)
    _close(y2, want_y, 1e-2)
    # fused quantisation == quantisation of the bf16 output it also wrote
    qr, sr = ref.act_quant(y2)
    assert torch.allclose(s2, sr, rtol=1e-6, atol=0)
    assert (q2.view(torch.uint8) != qr.view(torch.uint8)).float().mean().item() < 2e-3


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (77, 256, 1024), (300, 2112, 7168), (1024, 7168, 2048)])
def test_fp8_gemm(M, N, K):
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    xq, xs = ref.act_quant(x)
    wq, ws = ref.weight_quant_block(w)
    _close(gemm.fp8_gemm(xq, xs, wq, ws), ref.fp8_gemm(xq, xs, wq, ws))


@pytest.mark.parametrize("M,N,K", [(5, 128, 64), (200, 384, 512), (1000, 576, 7168)])
def test_bf16_gemm(M, N, K):
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    _close(gemm.bf16_gemm(x, w), x.float() @ w.float().t())


@pytest.mark.parametrize("M,N,K", [(3, 16, 1024), (150, 4096, 1024), (48, 129280, 7168)])
def test_bf16_gemm_fp32_epilogue(M, N, K):
    """fp32-output epilogue at the router shape and at lm_head shapes (many column tiles)."""
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    got = gemm.bf16_gemm(x, w, fp32_out=True)
    assert got.dtype == torch.float32
    want = x.float() @ w.float().t()
    torch.cuda.synchronize()
    err = (got - want).abs().max().item()
    assert err <= 2e-3 * want.abs().max().item(), (err, want.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(96, 2112, 7168), (384, 2112, 7168), (48, 7168, 2048), (96, 1536, 1536)])
def test_fp8_gemm_split_k_shapes(M, N, K):
    """Decode-sized projections: few output tiles, K split over several CTAs with an in-kernel reduction.  Two
    launches in a row (the per-tile counters must be back at zero) and bit-identical results (fixed summation order)."""
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    xq, xs = ref.act_quant(x)
    wq, ws = ref.weight_quant_block(w)
    want = ref.fp8_gemm(xq, xs, wq, ws)
    a = gemm.fp8_gemm(xq, xs, wq, ws, swapab=False)
    b = gemm.fp8_gemm(xq, xs, wq, ws, swapab=False)
    _close(a, want)
    assert torch.equal(a, b)


@pytest.mark.parametrize("M", [48, 384])
def test_router_gemm_split_k_fp32(M):
    x = torch.randn(M, 7168, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(256, 7168, device=DEV) * 0.05).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    a = gemm.bf16_gemm(x, w, fp32_out=True)
    b = gemm.bf16_gemm(x, w, fp32_out=True)
    torch.cuda.synchronize()
    assert (a - want).abs().max().item() <= 2e-3 * want.abs().max().item()
    assert torch.equal(a, b)


def test_fp8_gemm_fused_silu():
    M, I, K = 300, 256, 512
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(2 * I, K, device=DEV) * 0.05
    xq, xs = ref.act_quant(x)
    wq, ws = ref.weight_quant_block(w)
    perm = gemm.interleave_gate_up_rows(2 * I, DEV)
    y = gemm.fp8_gemm(xq, xs, wq.view(torch.uint8)[perm].contiguous().view(FP8), ws, silu_mul=True)
    _close(y, ref.silu_mul(ref.fp8_gemm(xq, xs, wq, ws)))


def test_grouped_fp8_gemm_ragged():
    E, N, K = 8, 512, 1024
    counts = torch.tensor([5, 0, 130, 128, 1, 300, 64, 17])
    padded = ((counts + 127) // 128) * 128
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(padded, 0)
    R = int(offs[-1])
    x = torch.randn(R, K, device=DEV)
    xq, xs = ref.act_quant(x)
    wq = torch.empty(E, N, K, device=DEV, dtype=FP8)
    ws = torch.empty(E, N // 128, K // 128, device=DEV)
    for e in range(E):
        wq[e], ws[e] = ref.weight_quant_block(torch.randn(N, K, device=DEV) * 0.05)
    y = gemm.grouped_fp8_gemm(xq, xs, wq, ws, offs.to(DEV))
    _close(y, ref.grouped_fp8_gemm(xq, xs, wq, ws, offs.to(DEV)))


# ---------------------------------------------------------------- swapped-operand FP8 GEMM (few rows per weight matrix)
@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (12, 256, 1024), (32, 2176, 7168), (45, 7168, 2048)])
def test_fp8_gemm_swapab_dense(M, N, K):
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    xq, xs = ref.act_quant(x)
    wq, ws = ref.weight_quant_block(w)
    _close(gemm.fp8_gemm(xq, xs, wq, ws, swapab=True), ref.fp8_gemm(xq, xs, wq, ws))


def _grouped_case(counts, N, K, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    E = len(counts)
    counts = torch.tensor(counts)
    padded = ((counts + 127) // 128) * 128
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(padded, 0)
    R = int(offs[-1])
    x = torch.randn(R, K, device=DEV, generator=g)
    xq, xs = ref.act_quant(x)
    wq = torch.empty(E, N, K, device=DEV, dtype=FP8)
    ws = torch.empty(E, N // 128, K // 128, device=DEV)
    for e in range(E):
        wq[e], ws[e] = ref.weight_quant_block(torch.randn(N, K, device=DEV, generator=g) * 0.05)
    real = torch.zeros(R, dtype=torch.bool)
    for e in range(E):
        real[int(offs[e]): int(offs[e]) + int(counts[e])] = True
    return xq, xs, wq, ws, offs.to(DEV), counts.to(torch.int32).to(DEV), real


def test_grouped_fp8_gemm_swapab_ragged():
    """Decode-shaped ragged groups: experts with no token, with a few, with more than one 32-token tile."""
    counts = [5, 0, 40, 12, 1, 33, 0, 17, 64, 9]
    xq, xs, wq, ws, offs, cnt, real = _grouped_case(counts, 512, 1024)
    y = gemm.grouped_fp8_gemm(xq, xs, wq, ws, offs, counts=cnt, rows_hint=sum(counts))
    want = ref.grouped_fp8_gemm(xq, xs, wq, ws, offs)
    torch.cuda.synchronize()
    _close(y[real.to(DEV)], want[real.to(DEV)])


def test_grouped_fp8_gemm_swapab_silu():
    counts = [7, 30, 0, 35]
    I, K = 256, 512
    xq, xs, wq, ws, offs, cnt, real = _grouped_case(counts, 2 * I, K, seed=1)
    perm = gemm.interleave_gate_up_rows(2 * I, DEV)
    wqi = wq.view(torch.uint8)[:, perm].contiguous().view(FP8)
    y = gemm.grouped_fp8_gemm(xq, xs, wqi, ws, offs, silu_mul=True, counts=cnt, rows_hint=sum(counts))
    want = ref.silu_mul(ref.grouped_fp8_gemm(xq, xs, wq, ws, offs))
    torch.cuda.synchronize()
    _close(y[real.to(DEV)], want[real.to(DEV)])


def test_swapab_and_tile_kernels_agree_on_experts_forward():
    """The whole expert stack of a decode-sized step (which selects the swapped-operand kernel) against the same step
    forced onto the token-major kernels."""
    import batchgen_b200.ops.gemm as G
    T, H, I, E, K = 48, 1024, 512, 16, 4
    g = torch.Generator(device=DEV).manual_seed(3)
    hidden = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, device=DEV, generator=g)
    w13 = torch.empty(E, 2 * I, H, device=DEV, dtype=FP8)
    w13s = torch.empty(E, 2 * I // 128, H // 128, device=DEV)
    w2 = torch.empty(E, H, I, device=DEV, dtype=FP8)
    w2s = torch.empty(E, H // 128, I // 128, device=DEV)
    for e in range(E):
        w13[e], w13s[e] = ref.weight_quant_block(torch.randn(2 * I, H, device=DEV, generator=g) * 0.05)
        w2[e], w2s[e] = ref.weight_quant_block(torch.randn(H, I, device=DEV, generator=g) * 0.05)
    ew = moe.ExpertWeights(w13=w13, w2=w2, w13_s=w13s, w2_s=w2s, quant="fp8_block").to_device_layout()
    old = G._SWAPAB
    try:
        G._SWAPAB = "1"
        a = moe.experts_forward(hidden, idx, w, ew, 0, E)
        G._SWAPAB = "0"
        b = moe.experts_forward(hidden, idx, w, ew, 0, E)
    finally:
        G._SWAPAB = old
    torch.cuda.synchronize()
    _close(a, b)


@pytest.mark.parametrize("E,K,ng,tg", [(256, 8, 8, 4), (256, 8, 1, 1), (896, 16, 1, 1), (64, 6, 4, 2)])
def test_router_sigmoid_topk(E, K, ng, tg):
    T = 200
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1
    idx, w = moe.router_topk(logits, bias, K, ng, tg, True, 2.5)
    ridx, rw = ref.router_topk(logits, bias, K, ng, tg, True, 2.5)
    a = torch.sort(idx, -1)[0]
    b = torch.sort(ridx, -1)[0]
    assert (a != b).any(-1).float().mean().item() < 0.01       # fp ties only
    same = (a == b).all(-1)
    so = torch.argsort(idx, -1)
    sr = torch.argsort(ridx, -1)
    assert torch.allclose(w.gather(1, so)[same], rw.gather(1, sr)[same], rtol=1e-4, atol=1e-6)


def test_router_softmax_topk():
    logits = torch.randn(64, 128, device=DEV)
    idx, w = moe.router_topk(logits, None, 4, scoring="softmax")
    ridx, rw = ref.router_topk(logits, None, 4, scoring="softmax")
    assert torch.equal(idx, ridx)
    assert torch.allclose(w, rw, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("scoring,E,K,ng,tg,norm", [("softmax_all", 160, 6, 8, 3, False), ("softmax_all", 64, 8, 1, 1, False),
                                                     ("sqrtsoftplus", 256, 6, 1, 1, True)])
def test_router_softmax_all_and_sqrtsoftplus(scoring, E, K, ng, tg, norm):
    T = 200
    logits = torch.randn(T, E, device=DEV) * 2
    bias = torch.randn(E, device=DEV) * 0.1 if scoring == "sqrtsoftplus" else None
    idx, w = moe.router_topk(logits, bias, K, ng, tg, norm, 1.5, scoring)
    ridx, rw = ref.router_topk(logits, bias, K, ng, tg, norm, 1.5, scoring)
    a, b = torch.sort(idx, -1)[0], torch.sort(ridx, -1)[0]
    assert (a != b).any(-1).float().mean().item() < 0.01       # fp ties only
    same = (a == b).all(-1)
    so, sr = torch.argsort(idx, -1), torch.argsort(ridx, -1)
    assert torch.allclose(w.gather(1, so)[same], rw.gather(1, sr)[same], rtol=1e-4, atol=1e-7)


def test_moe_permute_gather_combine_roundtrip():
    T, K, E, H = 333, 8, 64, 1024
    lo, hi = 16, 48
    idx = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, device=DEV)
    hidden = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    src, pos, offs = moe.permute(idx, lo, hi)
    o = offs.tolist()
    assert all(v % 128 == 0 for v in o)
    local = (idx >= lo) & (idx < hi)
    assert ((pos >= 0) == local).all()
    # every local pair lands in its expert's segment and points back at its token
    e_of = (idx - lo).clamp(0, hi - lo - 1).long()
    seg_lo = offs[:-1][e_of]
    seg_hi = offs[1:][e_of]
    assert ((pos >= seg_lo) & (pos < seg_hi))[local].all()
    tok = torch.arange(T, device=DEV).unsqueeze(1).expand(T, K)
    assert (src[pos[local].long()] == tok[local]).all()
    assert int((src[: o[-1]] >= 0).sum()) == int(local.sum())
    q, s = moe.gather_quant(hidden, src, offs)
    rows = ref.dequant_act(q[: o[-1]], s[: o[-1]].contiguous())
    want = torch.where((src[: o[-1]] >= 0).unsqueeze(-1), hidden[src[: o[-1]].clamp_min(0).long()].float(),
                       torch.zeros(1, device=DEV))
    _close(rows, want, 7e-2)
    y = torch.randn(src.shape[0], H, device=DEV, dtype=torch.bfloat16)
    extra = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    out = moe.combine(y, pos, w, extra)
    want = ref.moe_combine(y, pos.long(), w, torch.float32) + extra.float()
    _close(out, want, 1e-2)


def test_experts_forward_matches_reference():
    torch.manual_seed(1234)            # two quantisation steps sit between input and output: keep the draw fixed
    T, K, E, H, I = 150, 4, 16, 512, 256
    hidden = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, device=DEV)
    w13q = torch.empty(E, 2 * I, H, device=DEV, dtype=FP8)
    w13s = torch.empty(E, 2 * I // 128, H // 128, device=DEV)
    w2q = torch.empty(E, H, I, device=DEV, dtype=FP8)
    w2s = torch.empty(E, H // 128, I // 128, device=DEV)
    for e in range(E):
        w13q[e], w13s[e] = ref.weight_quant_block(torch.randn(2 * I, H, device=DEV) * 0.05)
        w2q[e], w2s[e] = ref.weight_quant_block(torch.randn(H, I, device=DEV) * 0.05)
    ew_ref = moe.ExpertWeights(w13q.cpu(), w2q.cpu(), w13s.cpu(), w2s.cpu(), quant="fp8_block")
    ew = moe.ExpertWeights(w13q.clone(), w2q, w13s, w2s, quant="fp8_block").to_device_layout()
    got = moe.experts_forward(hidden, idx, w, ew, 0, E)
    want = moe.experts_forward(hidden.cpu().float(), idx.cpu(), w.cpu(), ew_ref, 0, E)
    _close(got.cpu(), want, 4e-2)


def test_mla_kv_write_and_rope_q():
    T, kv_lora, rope, P, S = 90, 512, 64, 8, 64
    kv_a = torch.randn(T, kv_lora + rope + 100, device=DEV, dtype=torch.bfloat16)[:, 100:]
    w = (1 + 0.1 * torch.randn(kv_lora, device=DEV)).to(torch.bfloat16)
    pos = torch.randint(0, 4000, (T,), device=DEV, dtype=torch.int32)
    inv = ref.rope_inv_freq(rope, 10000.0, 40.0, 4096)
    ang = torch.arange(4096, dtype=torch.float32).unsqueeze(-1) * inv
    cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    slots = torch.randperm(P * S, device=DEV)[:T].to(torch.int64)
    slots[3] = -1
    for inter in (True, False):
        cache = torch.zeros(P, S, kv_lora + rope, device=DEV, dtype=torch.bfloat16)
        fused.mla_kv_write(kv_a, w, pos, cos, sin, slots, cache, kv_lora, 1e-6, inter)
        want = torch.zeros(P, S, kv_lora + rope, dtype=torch.float32)
        rows = ref.mla_kv_prepare(kv_a.float().cpu(), w.float().cpu(), cos[pos.long()].cpu(), sin[pos.long()].cpu(),
                                  kv_lora, 1e-6, inter)
        ref.kv_cache_write(want, rows, slots.cpu())
        _close(cache.cpu(), want, 1e-2)
        q = torch.randn(T, 16, 192, device=DEV, dtype=torch.bfloat16)
        q0 = q.clone()
        fused.rope_q_(q, pos, cos, sin, rope, inter)
        wantq = q0.float().cpu()
        wantq[..., -rope:] = ref.apply_rope(wantq[..., -rope:], cos[pos.long()].cpu(), sin[pos.long()].cpu(), inter)
        _close(q.cpu(), wantq, 1e-2)


def test_sampling_greedy_and_constraints():
    T, V = 64, 129280
    logits = torch.randn(T, V, device=DEV)
    assert torch.equal(sampling.greedy(logits).long(), logits.argmax(-1))
    assert torch.equal(sampling.greedy(logits.to(torch.bfloat16)).long(),
                       logits.to(torch.bfloat16).float().argmax(-1))
    temp = torch.full((T,), 0.8, device=DEV)
    temp[::4] = 0.0
    tk = torch.full((T,), 20, device=DEV, dtype=torch.int32)
    tp = torch.full((T,), 0.9, device=DEV)
    u = torch.rand(T, device=DEV)
    tok = sampling.sample(logits, temp, tk, tp, uniform=u).long()
    assert torch.equal(tok[::4], logits.argmax(-1)[::4])
    top20 = logits.topk(20, -1)[1]
    assert (tok.unsqueeze(-1) == top20).any(-1).all()
    # top_k = 1 is greedy whatever the temperature
    tok1 = sampling.sample(logits, torch.ones(T, device=DEV), torch.ones(T, device=DEV, dtype=torch.int32),
                           torch.ones(T, device=DEV), uniform=u).long()
    assert torch.equal(tok1, logits.argmax(-1))


def test_sampling_topk_then_topp_matches_reference_order():
    """Both filters active: the kernel's draw equals the sequential reference (top-k, then the nucleus of the
    renormalised survivors) for the same uniform numbers."""
    T, V = 96, 4096
    g = torch.Generator(device="cpu").manual_seed(3)
    logits = (torch.randn(T, V, generator=g) * 3.0).to(DEV)
    temp = torch.full((T,), 0.7, device=DEV)
    tk = torch.tensor([2, 5, 20, 50] * (T // 4), device=DEV, dtype=torch.int32)
    tp = torch.tensor([0.5, 0.8, 0.3] * (T // 3), device=DEV)
    u = torch.rand(T, generator=g).to(DEV)
    tok = sampling.sample(logits, temp, tk, tp, uniform=u).long().cpu()
    # kept set from the reference's sequential rule; the kernel's token must be inside it
    lf = logits.float().cpu() / 0.7
    sp, si = torch.sort(torch.softmax(lf, -1), -1, descending=True)
    for r in range(T):
        k = int(tk[r])
        sk = sp[r, :k]
        cum = torch.cumsum(sk, 0)
        keep = (cum - sk) <= float(tp[r]) * float(sk.sum())
        keep[0] = True
        allowed = set(si[r, :k][keep].tolist())
        assert int(tok[r]) in allowed, (r, int(tok[r]), sorted(allowed)[:8])
    # the example that separates the two semantics: p = (.3, .2, .1 x 5), k = 2, top_p = .5 keeps token 0 only
    p = torch.tensor([0.3, 0.2, 0.1, 0.1, 0.1, 0.1, 0.1], device=DEV)
    lg = p.log().unsqueeze(0).repeat(64, 1).contiguous()
    t2 = sampling.sample(lg, torch.ones(64, device=DEV), torch.full((64,), 2, device=DEV, dtype=torch.int32),
                         torch.full((64,), 0.5, device=DEV), uniform=torch.linspace(0, 0.999, 64, device=DEV))
    assert set(t2.tolist()) == {0}


def test_sampling_distribution():
    V, N = 50, 4000
    base = torch.randn(V, device=DEV)
    logits = base.unsqueeze(0).expand(N, V).contiguous()
    temp = torch.ones(N, device=DEV)
    tok = sampling.sample(logits, temp, torch.zeros(N, device=DEV, dtype=torch.int32), torch.ones(N, device=DEV),
                          uniform=torch.rand(N, device=DEV)).long()
    freq = torch.bincount(tok, minlength=V).float() / N
    assert (freq - torch.softmax(base, 0)).abs().max().item() < 0.03

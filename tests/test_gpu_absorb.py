"""Per-head batched GEMM (MLA absorb / out-absorb) and the grouped GEMM's real-row counts, against fp32
references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("T,H", [(1, 16), (200, 16), (384, 128), (130, 8)])
def test_q_absorb_and_out_absorb(T, H):
    from batchgen_b200.ops import _ext, attention
    g = torch.Generator().manual_seed(T + H)
    nope, rope, lora, v = 128, 64, 512, 128
    q = torch.randn(T, H, nope + rope, generator=g).to(torch.bfloat16).cuda()
    w_uk_t = (torch.randn(H, lora, nope, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w_uv = (torch.randn(H, v, lora, generator=g) * 0.05).to(torch.bfloat16).cuda()
    q_abs = attention.mla_q_absorb(q, w_uk_t, nope)
    _ext.check_status()
    want = torch.einsum("thk,hnk->thn", q[..., :nope].float(), w_uk_t.float())
    assert q_abs.shape == (T, H, lora) and _rel(q_abs, want) < 5e-3
    o_lat = torch.randn(T, H, lora, generator=g).to(torch.bfloat16).cuda()
    out = attention.mla_out_absorb(o_lat, w_uv)
    _ext.check_status()
    want = torch.einsum("thk,hnk->thn", o_lat.float(), w_uv.float()).reshape(T, H * v)
    assert out.shape == (T, H * v) and _rel(out, want) < 5e-3


def test_grouped_gemm_with_real_counts():
    from batchgen_b200.ops import _ext, gemm, ref
    FP8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(3)
    E, N, K = 4, 256, 256
    rows = [5, 0, 130, 128]
    starts, cur = [], 0
    for r in rows:
        starts.append(cur)
        cur += (r + 127) // 128 * 128
    offsets = torch.tensor(starts + [cur], dtype=torch.int32)
    x = torch.randn(cur, K, generator=g)
    xq, xs = ref.act_quant(x)
    wq = (torch.randn(E, N, K, generator=g) * 0.1).to(FP8)
    ws = torch.rand(E, N // 128, K // 128, generator=g) + 0.5
    counts = torch.tensor(rows, dtype=torch.int32).cuda()
    sentinel = 768.0
    out = torch.full((cur, N), sentinel, dtype=torch.bfloat16, device="cuda")
    xs_dev = xs.cuda().t().contiguous().t()
    gemm.grouped_fp8_gemm(xq.cuda(), xs_dev, wq.cuda(), ws.cuda(), offsets.cuda(), out=out, counts=counts)
    _ext.check_status()
    want = ref.grouped_fp8_gemm(xq, xs, wq, ws, offsets)
    out = out.cpu().float()
    for e in range(E):
        a, n = starts[e], rows[e]
        if n:
            assert _rel(out[a:a + n], want[a:a + n]) < 1e-2
        pad_end = offsets[e + 1].item()
        assert (out[a + n:pad_end] == sentinel).all(), "padding rows must not be stored"


@pytest.mark.parametrize("H", [4, 16])
def test_expanded_mla_prefill_attention(H):
    """Varlen causal attention over up-projected keys / values, with cached context on one sequence."""
    from batchgen_b200.ops import _ext, attention
    g = torch.Generator().manual_seed(H)
    lens, ctx = [300, 70, 129], [0, 200, 64]                 # new tokens and cached context per sequence
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    k_starts, tk = [], 0
    for n, c in zip(lens, ctx):
        k_starts.append(tk)
        tk += n + c
    Tq = cu[-1]
    q = (torch.randn(Tq, H, 192, generator=g) * 0.5).to(torch.bfloat16)
    kv = (torch.randn(tk, H, 256, generator=g) * 0.5).to(torch.bfloat16)
    lat = (torch.randn(tk, 576, generator=g) * 0.5).to(torch.bfloat16)
    kpe = lat[:, 512:]                                        # strided view, as the model passes it
    work = attention.mha_prefill_work(cu, ctx, k_starts)
    scale = 192 ** -0.5
    got = attention.mha_prefill(q.cuda(), kv.cuda(), lat.cuda()[:, 512:], work, scale).cpu().float()
    _ext.check_status()
    want = attention.mha_prefill(q.float(), kv.float(), kpe.float(), work, scale)
    assert _rel(got, want) < 1.5e-2


def test_model_prefill_uses_expanded_attention_and_matches_cpu():
    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.transformer import AttnMeta
    from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range
    cfg = get_model_config("tiny-deepseek-v3", hidden_size=1024, q_lora_rank=512, kv_lora_rank=512,
                           qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_heads=16,
                           intermediate_size=2048, moe_intermediate_size=512, n_routed_experts=16,
                           num_experts_per_tok=4, n_group=4, topk_group=2, vocab_size=4096, quant="fp8_block")
    lens = [330, 200]
    ids = torch.randint(2, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(5), dtype=torch.int32)

    def run(device, dtype_name, dtype):
        model = build_model(cfg, device, dtype_name, seed=0)
        kv = PagedKVCache(cfg, 16, 64, device, dtype)
        pages = [kv.alloc.alloc((n + 63) // 64) for n in lens]
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(device)
        slots = torch.tensor(sum((slots_for_range(p, 0, n, 64) for p, n in zip(pages, lens)), []), device=device)
        meta = AttnMeta(mode="prefill", positions=pos, slot_mapping=slots, block_table=build_block_table(pages, device),
                        cu_seqlens=[0, lens[0], sum(lens)], ctx_lens=[0, 0])
        return model, model.forward(ids.to(device), meta, kv).float().cpu()

    _, cpu = run("cpu", "fp32", torch.float32)
    model, gpu = run("cuda", "bf16", torch.bfloat16)
    assert model.w.layers[0].w_kvb is not None
    rel = ((gpu - cpu).norm() / cpu.norm()).item()
    assert rel < 0.08, rel


@pytest.mark.parametrize("T,N,K,silu", [(300, 512, 256, False), (128, 256, 128, False), (515, 768, 1024, True), (1, 2112, 7168, False)])
def test_wide_tile_fp8_gemm_matches_reference(T, N, K, silu):
    """128 x 256-tile kernel: same contract as the 128 x 128 one."""
    from batchgen_b200.ops import _ext, gemm, ref
    FP8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g)
    xq, xs = ref.act_quant(x)
    wq = (torch.randn(N, K, generator=g) * 0.1).to(FP8)
    ws = torch.rand((N + 127) // 128, K // 128, generator=g) + 0.5
    want = ref.fp8_gemm(xq, xs, wq, ws)
    wq_dev = wq.cuda()
    if silu:
        perm = gemm.interleave_gate_up_rows(N)
        wq_dev = wq.view(torch.uint8)[perm].contiguous().view(FP8).cuda()
        want = ref.silu_mul(want)
    xs_dev = xs.cuda().t().contiguous().t()
    got = gemm.fp8_gemm(xq.cuda(), xs_dev, wq_dev, ws.cuda(), silu_mul=silu, wide=True).cpu().float()
    narrow = gemm.fp8_gemm(xq.cuda(), xs_dev, wq_dev, ws.cuda(), silu_mul=silu, wide=False).cpu().float()
    _ext.check_status()
    assert _rel(got, want) < 1e-2
    # the narrow kernel may split K over CTAs at these sizes (a different but fixed summation order)
    assert _rel(narrow, want) < 1e-2 and _rel(got, narrow) < 2e-3


def test_wide_tile_grouped_gemm_with_counts():
    from batchgen_b200.ops import _ext, gemm, ref
    FP8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(11)
    E, N, K = 3, 512, 256
    rows = [130, 0, 7]
    starts, cur = [], 0
    for r in rows:
        starts.append(cur)
        cur += (r + 127) // 128 * 128
    offsets = torch.tensor(starts + [cur], dtype=torch.int32)
    xq, xs = ref.act_quant(torch.randn(cur, K, generator=g))
    wq = (torch.randn(E, N, K, generator=g) * 0.1).to(FP8)
    ws = torch.rand(E, N // 128, K // 128, generator=g) + 0.5
    out = torch.full((cur, N), 768.0, dtype=torch.bfloat16, device="cuda")
    gemm.grouped_fp8_gemm(xq.cuda(), xs.cuda().t().contiguous().t(), wq.cuda(), ws.cuda(), offsets.cuda(), out=out,
                          counts=torch.tensor(rows, dtype=torch.int32).cuda(), wide=True)
    _ext.check_status()
    want = ref.grouped_fp8_gemm(xq, xs, wq, ws, offsets)
    out = out.cpu().float()
    for e in range(E):
        a, n = starts[e], rows[e]
        if n:
            assert _rel(out[a:a + n], want[a:a + n]) < 1e-2
        assert (out[a + n:offsets[e + 1].item()] == 768.0).all()


def test_router_logits_fp32_epilogue():
    from batchgen_b200.ops import _ext, moe
    g = torch.Generator().manual_seed(9)
    x = torch.randn(300, 1024, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(256, 1024, generator=g) * 0.05).cuda()
    got = moe.router_logits(x, w)
    _ext.check_status()
    assert got.dtype == torch.float32 and got.shape == (300, 256)
    want = x.float() @ w.to(torch.bfloat16).float().t()
    assert _rel(got, want) < 1e-4
    # batch invariance: a row's logits do not depend on which other rows are in the batch
    assert torch.equal(moe.router_logits(x[:7].contiguous(), w), got[:7])

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

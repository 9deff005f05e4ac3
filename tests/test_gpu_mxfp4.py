"""MXFP4-weight tcgen05 GEMM against fp32 references of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def test_dequant_kernel_exact():
    from batchgen_b200.ops import mxfp4, ref
    w = torch.randn(96, 256) * 3
    q, s = mxfp4.quantize(w)
    d = mxfp4.dequantize(q.cuda(), s.cuda(), torch.float32).cpu()
    assert torch.equal(d, ref.mxfp4_dequant(q, s))


@pytest.mark.parametrize("T,N,K", [(128, 128, 64), (200, 384, 512), (1, 7168, 3584), (515, 200, 1024)])
def test_dense_gemm(T, N, K):
    from batchgen_b200.ops import _ext, mxfp4
    g = torch.Generator().manual_seed(T + N)
    w = torch.randn(N, K, generator=g) * 0.05
    q, s = mxfp4.quantize(w)
    x = (torch.randn(T, K, generator=g)).to(torch.bfloat16)
    y = mxfp4.mxfp4_gemm(x.cuda(), q.cuda(), s.cuda())
    _ext.check_status()
    want = x.float() @ mxfp4.dequantize(q, s, torch.float32).t()
    assert _rel(y.cpu(), want) < 6e-3


@pytest.mark.parametrize("silu", [False, True])
def test_grouped_gemm(silu):
    from batchgen_b200.ops import _ext, mxfp4
    from batchgen_b200.ops.gemm import interleave_gate_up_rows
    g = torch.Generator().manual_seed(5)
    E, N, K = 5, 256, 384
    rows = [128, 0, 37, 256, 1]
    starts, cur = [0], 0
    for r in rows:
        cur += (r + 127) // 128 * 128
        starts.append(cur)
    offsets = torch.tensor([starts[i] for i in range(E)] + [starts[-1]], dtype=torch.int32)
    # segment e holds rows[e] real rows followed by padding up to the next 128-aligned start
    ends = [starts[e] + rows[e] for e in range(E)]
    x = torch.zeros(starts[-1], K)
    for e in range(E):
        x[starts[e]:ends[e]] = torch.randn(rows[e], K, generator=g)
    x = x.to(torch.bfloat16)
    w = torch.randn(E, N, K, generator=g) * 0.05
    q, s = mxfp4.quantize(w)
    wd = mxfp4.dequantize(q, s, torch.float32)
    qd, sd = q.cuda(), s.cuda()
    if silu:
        perm = interleave_gate_up_rows(N)
        qd, sd = qd[:, perm.cuda()].contiguous(), sd[:, perm.cuda()].contiguous()
    y = mxfp4.grouped_mxfp4_gemm(x.cuda(), qd, sd, offsets.cuda(), silu_mul=silu).cpu()
    _ext.check_status()
    for e in range(E):
        if rows[e] == 0:
            continue
        ref_e = x[starts[e]:ends[e]].float() @ wd[e].t()
        if silu:
            ref_e = torch.nn.functional.silu(ref_e[:, : N // 2]) * ref_e[:, N // 2:]
        assert _rel(y[starts[e]:ends[e]], ref_e) < 8e-3, e


@pytest.mark.parametrize("silu", [False, True])
def test_int4_grouped_gemm(silu):
    from batchgen_b200.ops import _ext, int4
    from batchgen_b200.ops.gemm import interleave_gate_up_rows
    g = torch.Generator().manual_seed(8)
    E, N, K = 3, 256, 256
    rows = [130, 0, 5]
    starts, cur = [], 0
    for r in rows:
        starts.append(cur)
        cur += (r + 127) // 128 * 128
    offsets = torch.tensor(starts + [cur], dtype=torch.int32)
    x = torch.randn(cur, K, generator=g).to(torch.bfloat16)
    q, s = int4.quantize(torch.randn(E, N, K, generator=g) * 0.05)
    wd = int4.dequantize(q, s)
    qd, sd = q.cuda(), s.cuda()
    if silu:
        perm = interleave_gate_up_rows(N).cuda()
        qd, sd = qd[:, perm].contiguous(), sd[:, perm].contiguous()
    y = int4.grouped_int4_gemm(x.cuda(), qd, sd, offsets.cuda(), silu_mul=silu).cpu()
    _ext.check_status()
    for e in range(E):
        a, n = starts[e], rows[e]
        if not n:
            continue
        want = x[a:a + n].float() @ wd[e].t()
        if silu:
            want = torch.nn.functional.silu(want[:, : N // 2]) * want[:, N // 2:]
        assert _rel(y[a:a + n], want) < 8e-3, e
    assert _rel(int4.int4_gemm(x[:40].cuda(), q[0].cuda(), s[0].cuda()).cpu(), x[:40].float() @ wd[0].t()) < 8e-3

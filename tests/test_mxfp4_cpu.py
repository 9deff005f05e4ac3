"""MXFP4 expert path on CPU: quantiser, dequantiser, grouped expert stack, a model built with MXFP4 experts."""
import torch

from batchgen_b200.ops import moe, mxfp4, ref


def test_quant_dequant_roundtrip():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(48, 128, generator=g)
    q, s = mxfp4.quantize(w)
    assert q.shape == (48, 64) and s.shape == (48, 4) and q.dtype == torch.uint8
    d = mxfp4.dequantize(q, s, torch.float32)
    # e2m1 has a 1-bit mantissa: relative error of a block's largest element is at most 1/4 step of 6
    assert (d - w).abs().max() <= (w.abs().amax() / 6.0) * 1.01
    q2, s2 = mxfp4.quantize(d)                      # representable values survive a second pass unchanged
    assert torch.equal(mxfp4.dequantize(q2, s2, torch.float32), d)


def test_grouped_experts_match_dequantised_dense():
    g = torch.Generator().manual_seed(1)
    E, I, K, Hout = 3, 64, 128, 128
    w13 = torch.randn(E, 2 * I, K, generator=g) * 0.1
    w2 = torch.randn(E, Hout, I, generator=g) * 0.1
    q13, s13 = mxfp4.quantize(w13)
    q2, s2 = mxfp4.quantize(w2)
    ew = moe.ExpertWeights(w13=q13, w2=q2, w13_s=s13, w2_s=s2, quant="mxfp4")
    dense = moe.ExpertWeights(w13=mxfp4.dequantize(q13, s13, torch.float32), w2=mxfp4.dequantize(q2, s2, torch.float32))
    x = torch.randn(10, K, generator=g)
    offsets = torch.tensor([0, 4, 4, 10], dtype=torch.int32)
    a = moe.grouped_experts(None, None, offsets, ew, x_dense=x)
    b = moe.grouped_experts(None, None, offsets, dense, x_dense=x)
    assert torch.allclose(a, b, atol=1e-5, rtol=1e-5)


def test_model_with_mxfp4_experts_runs():
    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.transformer import AttnMeta
    from batchgen_b200.runtime.kv_cache import PagedKVCache
    cfg = get_model_config("tiny-kimi-k3", quant="mxfp4", quant_block=32)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=3)
    lw = next(l for l in model.w.layers if l.experts is not None)
    assert lw.experts.quant == "mxfp4" and lw.experts.w13.dtype == torch.uint8
    kv = PagedKVCache(cfg, num_pages=8, page_size=16, device="cpu", dtype=torch.float32)
    T = 12
    ids = torch.arange(T, dtype=torch.int32) % cfg.vocab_size
    meta = AttnMeta(mode="prefill", positions=torch.arange(T, dtype=torch.int32),
                    slot_mapping=torch.arange(T, dtype=torch.int64), block_table=torch.arange(1, dtype=torch.int32).view(1, 1),
                    cu_seqlens=[0, T], ctx_lens=[0], logit_rows=torch.tensor([T - 1]))
    logits = model.forward(ids, meta, kv)
    assert logits.shape[-1] == cfg.vocab_size and torch.isfinite(logits).all()


def test_int4_quantiser_and_expert_stack_on_cpu():
    from batchgen_b200.ops import int4
    g = torch.Generator().manual_seed(2)
    w = torch.randn(3, 128, 128, generator=g) * 0.1
    q, s = int4.quantize(w)
    assert q.shape == (3, 128, 64) and s.shape == (3, 128, 4) and s.dtype == torch.bfloat16
    d = int4.dequantize(q, s)
    assert (d - w).abs().max() <= w.abs().max() / 7.0 * 0.6
    q13, s13 = int4.quantize(torch.randn(3, 128, 128, generator=g) * 0.1)
    q2, s2 = int4.quantize(torch.randn(3, 128, 64, generator=g) * 0.1)
    ew = moe.ExpertWeights(w13=q13, w2=q2, w13_s=s13, w2_s=s2, quant="int4")
    dense = moe.ExpertWeights(w13=int4.dequantize(q13, s13), w2=int4.dequantize(q2, s2))
    x = torch.randn(9, 128, generator=g)
    offsets = torch.tensor([0, 2, 2, 9], dtype=torch.int32)
    a = moe.grouped_experts(None, None, offsets, ew, x_dense=x)
    b = moe.grouped_experts(None, None, offsets, dense, x_dense=x)
    assert torch.allclose(a, b, atol=1e-5, rtol=1e-5)


def test_model_with_int4_experts_runs():
    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    cfg = get_model_config("tiny-kimi-k3", quant="int4", quant_block=32)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=3)
    lw = next(l for l in model.w.layers if l.experts is not None)
    assert lw.experts.quant == "int4" and lw.experts.w13_s.dtype == torch.bfloat16

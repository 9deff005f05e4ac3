#!/usr/bin/env python
"""Micro-benchmarks of the individual sm_100a kernels with roofline fractions.

    python benchmarks/kernel_bench.py <case> [--iters N] [size flags]

Cases: gemm_fp8, gemm_bf16, grouped_fp8, mla_decode, mla_prefill, mha_prefill, kda_decode, kda_prefill, norm_quant.  Each case uses inputs
larger than the 126 MB L2, warms up, times with CUDA events on the launching stream and prints one JSON
line: time, achieved TFLOP/s or GB/s, and the fraction "of measured" peak (MEASURED_PEAKS.json at the
repository root when present, else the fallback figures 6.65 TB/s / 1.59 PFLOP/s, "of fallback").
The same command lines are the ones profiled with ncu for the summaries under profiles/.

``--impl`` selects what is timed on the same inputs: ``ours`` (this repository's kernel), or a library anchor —
``flashinfer`` for ``mla_decode`` (``flashinfer.mla.trtllm_batch_decode_with_kv_cache_mla`` on the trtllm-gen
backend, called the way the reference calls it on Blackwell, batchgen/attention/mla/trtllm_gen_mla.py:49-93) and
``torch`` / ``vllm`` for ``gemm_fp8`` (cuBLASLt through ``torch._scaled_mm`` with 1x128 / 128x128 block scales where
the build supports them, else row-wise scales, else a bf16 ``torch.matmul``; vLLM's CUTLASS block-scaled GEMM).  A
library anchor is not the reference itself; it is the kernel the reference (or a stock serving stack) would call on
this GPU.  The output names which variant really ran.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from batchgen_b200.ops import _ext, fused, gemm, ref  # noqa: E402
from batchgen_b200.ops.mla_kernel import mla_decode_tc, mla_prefill_tc  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_CLOCK = {}


def sm_clock_mhz():
    """Current SM clock of device 0 (read through NVML; reading changes nothing), or None."""
    try:
        import pynvml
        if "h" not in _CLOCK:
            pynvml.nvmlInit()
            _CLOCK["h"] = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        return int(pynvml.nvmlDeviceGetClockInfo(_CLOCK["h"], pynvml.NVML_CLOCK_SM))
    except Exception:  # noqa: BLE001
        return None


SPIN_SECONDS = 0.4


def spin_up(seconds=None):
    """Keep the GPU busy for a while before a short kernel is timed: an idle B200 sits at a few hundred MHz and takes
    tens of milliseconds to raise its clocks, so a microsecond-scale kernel timed cold runs at a fraction of the
    clock it sees inside a real step."""
    seconds = SPIN_SECONDS if seconds is None else seconds
    if seconds <= 0:
        return
    a = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    e = torch.cuda.Event(enable_timing=True)
    s0 = torch.cuda.Event(enable_timing=True)
    s0.record()
    while True:
        for _ in range(20):
            a @ a
        e.record()
        e.synchronize()
        if s0.elapsed_time(e) >= seconds * 1e3:
            break


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    spin_up()
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    _CLOCK["mhz"] = sm_clock_mhz()          # sampled while the timed launches are still running or just done
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


_FI_WS = {}


def flashinfer_mla_decode(q, cache, bt, sl, max_len, scale):
    """The reference's Blackwell MLA decode call (dense form): absorbed query [B, 1, H, 576], latent cache
    [P, 64, 576], one zero-initialised 128 MiB workspace per device that every call reuses."""
    from flashinfer.mla import trtllm_batch_decode_with_kv_cache_mla
    B, H, W = q.shape
    ws = _FI_WS.setdefault(q.device.index, torch.zeros(128 * 1024 * 1024, dtype=torch.uint8, device=q.device))
    q4 = q.view(B, 1, H, W)

    def run():
        return trtllm_batch_decode_with_kv_cache_mla(
            query=q4, kv_cache=cache, workspace_buffer=ws, qk_nope_head_dim=512, kv_lora_rank=512,
            qk_rope_head_dim=W - 512, block_tables=bt, seq_lens=sl.clamp(min=1), max_seq_len=int(max_len),
            sparse_mla_top_k=0, bmm1_scale=float(scale), bmm2_scale=1.0, backend="trtllm-gen")
    run()
    return run


def library_fp8_gemm(impl, xq, xs, wq, ws):
    """-> (callable, name of the variant that ran).  xq [M, K] e4m3 with 1x128 scales xs [M, K/128] (a transposed view of
    a [K/128, M] buffer), wq [N, K] e4m3 with 128x128 scales ws [N/128, K/128]."""
    M, K = xq.shape
    N = wq.shape[0]
    tried = []
    if impl == "vllm":
        from vllm import _custom_ops as vops
        sa = xs                                                # [M, K/128], M-major (a view of the [K/128, M] buffer)
        sb = ws.t()                                            # [K/128, N/128] view of the [N/128, K/128] scales
        fn = lambda: vops.cutlass_scaled_mm(xq, wq.t(), sa, sb, torch.bfloat16)
        fn()
        return fn, "vllm cutlass_scaled_mm, 1x128 / 128x128 block scales"
    # torch._scaled_mm: block scales first (1x128 activations, 128x128 weights), then row-wise, then bf16
    for name, sa, sb in (
            ("torch._scaled_mm (cuBLASLt), 1x128 / 128x128 block scales", xs.t().contiguous().t(), ws.t().contiguous()),
            ("torch._scaled_mm (cuBLASLt), 1x128 / 128x128 block scales (row-major scale_a)", xs.contiguous(),
             ws.t().contiguous()),
            ("torch._scaled_mm (cuBLASLt), row-wise scales (coarser than the block scales of ours)",
             xs[:, :1].contiguous(), ws[:1, :1].expand(1, N).contiguous())):
        try:
            fn = lambda sa=sa, sb=sb: torch._scaled_mm(xq, wq.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
            fn()
            torch.cuda.synchronize()
            return fn, name
        except Exception as e:  # noqa: BLE001
            tried.append(f"{name}: {type(e).__name__}: {str(e)[:120]}")
    xb, wb = xq.to(torch.bfloat16), wq.to(torch.bfloat16)
    fn = lambda: torch.matmul(xb, wb.t())
    fn()
    return fn, "torch.matmul bf16 (cuBLAS); FP8 library variants failed: " + " | ".join(tried)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--rows", type=int, default=128, help="rows per expert (grouped)")
    ap.add_argument("--batch", type=int, default=96)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--spin", type=float, default=0.4, help="seconds of GEMM load before timing (0 under a profiler)")
    ap.add_argument("--impl", default="ours", choices=["ours", "flashinfer", "torch", "vllm"])
    ap.add_argument("--check", action="store_true", help="also compare the library result with this repository's")
    a = ap.parse_args()
    global SPIN_SECONDS
    SPIN_SECONDS = a.spin
    dev = "cuda"
    hbm, tf, tag = peaks()
    out = {"case": a.case}
    if a.case in ("gemm_fp8", "gemm_bf16"):
        M, N, K = a.m, a.n, a.k
        if a.case == "gemm_fp8":
            xq = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
            wq = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn)
            xs = torch.rand(K // 128, M, device=dev).t()
            ws = torch.rand((N + 127) // 128, K // 128, device=dev)
            if a.impl == "ours":
                ms = timeit(lambda: gemm.fp8_gemm(xq, xs, wq, ws), a.iters)
            else:
                fn, variant = library_fp8_gemm(a.impl, xq, xs, wq, ws)
                out["impl"] = variant
                ms = timeit(fn, a.iters)
                if a.check:
                    want = gemm.fp8_gemm(xq, xs, wq, ws).float()
                    got = fn().float()
                    out["rel_vs_ours"] = float((got - want).norm() / want.norm())
            byts = M * K + N * K + M * N * 2
        else:
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: gemm.bf16_gemm(x, w), a.iters)
            byts = 2 * (M * K + N * K + M * N)
        fl = 2.0 * M * N * K
        out.update(shape=[M, N, K], ms=ms, tflops=fl / ms / 1e9, frac_of_bf16_gemm_peak=fl / ms / 1e9 / tf,
                   gbs=byts / ms / 1e6, peak_note=tag)
    elif a.case == "grouped_fp8":
        E, N, K, R = a.experts, a.n, a.k, a.rows
        pad = (R + 127) // 128 * 128
        offs = (torch.arange(E + 1, dtype=torch.int32) * pad).to(dev)
        xq = torch.randn(E * pad, K, device=dev).to(torch.float8_e4m3fn)
        xs = torch.rand(K // 128, E * pad, device=dev).t()
        wq = torch.randn(E, N, K, device=dev).to(torch.float8_e4m3fn)
        ws = torch.rand(E, N // 128, K // 128, device=dev)
        cnt = torch.full((E,), R, dtype=torch.int32, device=dev)          # real rows per expert; the rest is padding
        ms = timeit(lambda: gemm.grouped_fp8_gemm(xq, xs, wq, ws, offs, counts=cnt, rows_hint=E * R), a.iters)
        byts = E * N * K + E * R * K + E * R * N * 2
        out.update(shape=[E, R, N, K], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm,
                   tflops=2.0 * E * pad * N * K / ms / 1e9, peak_note=tag)
    elif a.case in ("mla_decode", "mla_prefill"):
        B, H, L = a.batch, a.heads, a.ctx
        S = 64
        npg = (L + S - 1) // S
        if a.case == "mla_decode":
            cache = (torch.randn(B * npg, S, 576, device=dev) * 0.5).to(torch.bfloat16)
            bt = torch.arange(B * npg, dtype=torch.int32, device=dev).view(B, npg)
            q = torch.randn(B, H, 576, device=dev).to(torch.bfloat16)
            qa, qp = q[..., :512].contiguous(), q[..., 512:].contiguous()
            sl = torch.full((B,), L, dtype=torch.int32, device=dev)
            if a.impl == "ours":
                ms = timeit(lambda: mla_decode_tc(qa, qp, cache, bt, sl, 0.1, 512), a.iters)
            else:
                fn = flashinfer_mla_decode(q, cache, bt, sl, L, 0.1)
                out["impl"] = "flashinfer.mla.trtllm_batch_decode_with_kv_cache_mla (trtllm-gen)"
                ms = timeit(fn, a.iters)
                if a.check:
                    want = mla_decode_tc(qa, qp, cache, bt, sl, 0.1, 512).float()
                    got = fn().view(B, H, 512).float()
                    out["rel_vs_ours"] = float((got - want).norm() / want.norm())
            byts = B * L * 1152
            fl = 2.0 * B * L * H * (576 + 512)
        else:
            cache = (torch.randn(B * npg, S, 576, device=dev) * 0.5).to(torch.bfloat16)
            bt = torch.arange(B * npg, dtype=torch.int32, device=dev).view(B, npg)
            q = torch.randn(B * L, H, 576, device=dev).to(torch.bfloat16)
            qa, qp = q[..., :512].contiguous(), q[..., 512:].contiguous()
            cu = [i * L for i in range(B + 1)]
            ms = timeit(lambda: mla_prefill_tc(qa, qp, cache, bt, cu, [0] * B, 0.1, 512), a.iters)
            byts = B * L * 1152
            fl = 2.0 * B * (L * (L + 1) / 2) * H * (576 + 512)
        out.update(shape=[B, H, L], ms=ms, kv_gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm,
                   tflops=fl / ms / 1e9, frac_of_bf16_gemm_peak=fl / ms / 1e9 / tf, peak_note=tag)
    elif a.case == "mha_prefill":
        from batchgen_b200.ops import attention as attn_ops
        B, H, L = a.batch, a.heads, a.ctx
        T = B * L
        q = torch.randn(T, H, 192, device=dev).to(torch.bfloat16)
        kv = torch.randn(T, H, 256, device=dev).to(torch.bfloat16)
        kpe = torch.randn(T, 64, device=dev).to(torch.bfloat16)
        cu = [i * L for i in range(B + 1)]
        work = attn_ops.mha_prefill_work(cu, [0] * B, cu[:-1]).to(dev)
        ms = timeit(lambda: attn_ops.mha_prefill(q, kv, kpe, work, 0.07), a.iters)
        fl = 2.0 * B * (L * (L + 1) / 2) * H * (192 + 128)
        out.update(shape=[B, H, L], ms=ms, tflops=fl / ms / 1e9, frac_of_bf16_gemm_peak=fl / ms / 1e9 / tf, peak_note=tag)
    elif a.case in ("kda_decode", "kda_prefill"):
        from batchgen_b200.ops import kda
        B, H, D = a.batch, a.heads, 128
        L = 1 if a.case == "kda_decode" else a.ctx
        T, HD = B * L, H * D
        wide = torch.randn(T, 4 * HD + 8, device=dev).to(torch.bfloat16)
        f = torch.randn(T, HD, device=dev).to(torch.bfloat16)
        p = kda.KDAParams(torch.randn(3 * HD, 4, device=dev) * 0.5, None, torch.zeros(H, device=dev),
                          torch.zeros(HD, device=dev), torch.ones(D, device=dev))
        conv = torch.zeros(B, 3 * HD, 3, device=dev)
        rec = torch.zeros(B, H, D, D, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        cu = None if L == 1 else torch.arange(B + 1, dtype=torch.int32, device=dev) * L
        ms = timeit(lambda: kda.kda_forward(wide[:, : 3 * HD], f, wide[:, 4 * HD: 4 * HD + H], wide[:, 3 * HD: 4 * HD], p,
                                            conv, rec, slots, cu, None, H, D, D ** -0.5, 1e-6), a.iters)
        byts = 2 * B * H * D * D * 4 + T * HD * 2 * 6
        out.update(shape=[B, H, L], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm,
                   us_per_token=ms * 1e3 / L, peak_note=tag)
    elif a.case == "norm_quant":
        T, H = a.m, 7168
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        r = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: fused.rmsnorm(x, w, 1e-6, residual=r, quant=True), a.iters)
        byts = T * H * (2 + 2 + 2 + 2 + 1)
        out.update(shape=[T, H], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm, peak_note=tag)
    else:
        raise SystemExit(f"unknown case {a.case}")
    _ext.check_status()
    out["sm_mhz_at_timing"] = _CLOCK.get("mhz")
    print(json.dumps(out))


if __name__ == "__main__":
    main()

"""The allocation-free split-KV MLA decode entry point (``bg_mla_decode_split_noalloc``).

Some users of the kernel library cannot allocate device memory when they need attention computed:
code between the begin and end of a stream capture, serving loops that must never take the allocator
lock or synchronise the device, and embedders whose memory budget was fixed at start-up.  For them
the library exports one C entry point whose split-KV scratch, work list and merge list live in a
fixed device array inside the library (about 16.9 MB per GPU, at most 256 CTAs of work).

This test calls that exported C symbol through ctypes -- not through the package's wrappers -- twice
in a row, and compares each result with the regular entry point (caller-provided scratch) on the same
inputs.  It is collected last so that a run that stops at the first failure has run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(lens, H, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    S = 64
    need = [(l + S - 1) // S for l in lens]
    P = sum(need) + 2
    cache = (torch.randn(P, S, 576, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(P, device=DEV, generator=g).to(torch.int32)
    bt = torch.zeros(len(lens), max(need) + 1, dtype=torch.int32, device=DEV)
    o = 0
    for i, n in enumerate(need):
        bt[i, :n] = perm[o:o + n]
        o += n
    q = torch.randn(len(lens), H, 576, device=DEV, generator=g).to(torch.bfloat16)
    return cache, bt, q[..., :512].contiguous(), q[..., 512:].contiguous(), torch.tensor(lens, dtype=torch.int32,
                                                                                         device=DEV)


def _call_noalloc(lib, q_abs, q_pe, cache, bt, sl, splits, scale, status=None):
    B, H, _ = q_abs.shape
    out = torch.empty(B, H, 512, dtype=torch.bfloat16, device=DEV)
    P, S, D = cache.shape
    fn = lib.bg_mla_decode_split_noalloc
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(q_abs.data_ptr()), ctypes.c_void_p(q_pe.data_ptr()), ctypes.c_longlong(q_pe.stride(1)),
            ctypes.c_int(B), ctypes.c_int(H), ctypes.c_void_p(cache.data_ptr()), ctypes.c_longlong(P * S),
            ctypes.c_void_p(bt.data_ptr()), ctypes.c_int(bt.stride(0)), ctypes.c_void_p(sl.data_ptr()),
            ctypes.c_void_p(out.data_ptr()), ctypes.c_int(splits), ctypes.c_float(scale),
            ctypes.c_void_p(0 if status is None else status.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    from batchgen_b200.ops import _ext
    from batchgen_b200.ops.mla_kernel import mla_decode_tc
    lib = _ext.lib()
    lib.bg_noalloc_strerror.restype = ctypes.c_char_p
    # 16 and 32 heads fill their column variant; 8 and 24 heads run 8 heads per group on the 16-column variant with
    # half of the columns unused
    cases = [([1000, 130, 64, 2500], 16, 4), ([777, 90, 1300], 32, 3), ([900, 70, 2100], 8, 4), ([400, 1500], 24, 3)]
    status = _ext.status_word(DEV)
    for call, (lens, H, splits) in enumerate(cases):
        cache, bt, q_abs, q_pe, sl = _inputs(lens, H, seed=10 + call)
        rc, got = _call_noalloc(lib, q_abs, q_pe, cache, bt, sl, splits, 0.07, status=status if call % 2 else None)
        assert rc == 0, lib.bg_noalloc_strerror(rc)
        want = mla_decode_tc(q_abs, q_pe, cache, bt, sl, 0.07, 512, num_splits=splits)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        scale = want.float().abs().max().item()
        assert err <= 2e-2 * scale, (call, err, scale)
    _ext.check_status()


def test_noalloc_entry_point_rejects_oversized_problems():
    from batchgen_b200.ops import _ext
    lib = _ext.lib()
    lib.bg_noalloc_strerror.restype = ctypes.c_char_p
    cache, bt, q_abs, q_pe, sl = _inputs([64] * 40, 16, seed=3)
    rc, _ = _call_noalloc(lib, q_abs, q_pe, cache, bt, sl, 8, 0.1)       # 40 * 1 * 8 = 320 > 256
    assert rc == -20
    assert b"256" in lib.bg_noalloc_strerror(rc)
    rc, _ = _call_noalloc(lib, q_abs, q_pe, cache, bt, sl, 1, 0.1)       # the split path needs >= 2 splits
    assert rc == -21

"""Failure detection on the GPU without faulting it: a device-side wait on a flag that nothing raises runs
out of its (short) budget, the kernel returns, the host reads the status word, and the context keeps working."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_context_survives():
    from batchgen_b200.ops import _ext, gemm
    from batchgen_b200.parallel.fused import bounded_flag_wait
    dev = torch.device("cuda", 0)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    _ext.status_word(dev).zero_()
    t0 = time.perf_counter()
    bounded_flag_wait(flags, 2, epoch=5, budget_ms=300)          # nothing ever writes 5
    with pytest.raises(_ext.KernelError):
        _ext.check_status(dev)                                    # synchronises; status 4 = peer wait expired
    dt = time.perf_counter() - t0
    assert 0.25 < dt < 5.0, dt
    # the status word was cleared by check_status; a satisfied wait and an ordinary kernel still run
    flags.fill_(7)
    bounded_flag_wait(flags, 2, epoch=5, budget_ms=300)
    x = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    y = gemm.bf16_gemm(x, x)
    assert _ext.check_status(dev) == 0
    assert torch.isfinite(y.float()).all()


def test_later_waits_drain_quickly_once_status_is_raised():
    from batchgen_b200.ops import _ext
    from batchgen_b200.parallel.fused import bounded_flag_wait
    dev = torch.device("cuda", 0)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    _ext.status_word(dev).zero_()
    bounded_flag_wait(flags, 1, epoch=9, budget_ms=200)
    t0 = time.perf_counter()
    for _ in range(20):                                           # would be 20 x 2 s if each ran out its own budget
        bounded_flag_wait(flags, 1, epoch=9, budget_ms=2000)
    with pytest.raises(_ext.KernelError):
        _ext.check_status(dev)
    assert time.perf_counter() - t0 < 3.0

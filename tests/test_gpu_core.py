"""Native engine on the GPU: weight ring with the CUDA copy backend, KV page movers both ways."""
import pytest
import torch

from batchgen_b200.core import native

pytestmark = pytest.mark.gpu


def test_weight_ring_cuda_backend_streams_pinned_experts():
    ring = native.WeightRing(num_slots=3, slot_bytes=8 << 20, device="cuda:0")
    mods = {}
    for i in range(6):
        mods[f"e{i}"] = {"w13": torch.randn(512, 1024).bfloat16().pin_memory(),
                         "w2": torch.randn(1024, 256).bfloat16().pin_memory()}
        ring.register(f"e{i}", mods[f"e{i}"])
    order = list(mods)
    ring.install_queue(order)
    ring.start()
    x = torch.randn(4, 1024, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        ring.begin_pass(carry=True)
        for k in order:
            w = ring.get(k, timeout_ms=10000)
            assert w is not None and w["w13"].is_cuda
            y = x @ w["w13"].t()                              # consume on the compute stream
            assert torch.equal(w["w13"].cpu(), mods[k]["w13"]) and torch.equal(w["w2"].cpu(), mods[k]["w2"])
            ring.release(k, stream)                           # asynchronous release on a stream event
            assert y.shape == (4, 512)
        assert ring.end_pass()
    st = ring.stats()
    assert st["modules_copied"] == 12 and st["stalls"] == 0 and st["bytes_copied"] == 12 * (512 * 1024 + 1024 * 256) * 2
    ring.stop()
    ring.close()


@pytest.mark.parametrize("use_kernel", [True, False])
def test_kv_mover_host_to_device_and_back(use_kernel):
    kv = native.HostPagedKV(num_pages=16, page_bytes=64 * 576 * 2, prefix_slots=0)
    assert kv.pin()
    mover = native.KVMover(0, max_fragments=64)
    dev = torch.zeros(16, 64, 576, device="cuda", dtype=torch.bfloat16)
    host_pages = kv.alloc(5)
    for p in host_pages:
        kv.page_tensor(p, torch.bfloat16).copy_(torch.randn(64 * 576).bfloat16())
    dst = [3, 9, 1, 14, 7]
    nbytes = 64 * 576 * 2
    t = mover.submit([kv.page_ptr(p) for p in host_pages], [dev[d].data_ptr() for d in dst], nbytes, use_kernel)
    mover.stream_wait(t, torch.cuda.current_stream().cuda_stream)
    mover.wait(t)
    assert mover.done(t)
    for p, d in zip(host_pages, dst):
        assert torch.equal(dev[d].cpu().view(-1), kv.page_tensor(p, torch.bfloat16))
    # device -> host (offload), ordered after work on the compute stream
    dev[2].normal_()
    back = kv.alloc(1)
    t2 = mover.submit([dev[2].data_ptr()], [kv.page_ptr(back[0])], nbytes, use_kernel,
                      after_stream=torch.cuda.current_stream().cuda_stream)
    mover.wait(t2)
    assert torch.equal(dev[2].cpu().view(-1), kv.page_tensor(back[0], torch.bfloat16))
    assert mover.bytes_moved == 6 * nbytes
    mover.close()
    kv.close()

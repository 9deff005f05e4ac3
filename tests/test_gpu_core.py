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


def test_streamed_fp8_experts_match_resident_on_gpu():
    """FP8 experts parked in pinned host memory and streamed through the CUDA weight ring: same logits as the
    resident model, every MoE layer copied once per pass, slots released on the consumer stream."""
    import torch

    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.transformer import AttnMeta
    from batchgen_b200.ops import _ext
    from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range
    cfg = get_model_config("tiny-deepseek-v3", hidden_size=1024, q_lora_rank=512, kv_lora_rank=512,
                           qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_heads=16,
                           intermediate_size=2048, moe_intermediate_size=512, n_routed_experts=16,
                           num_experts_per_tok=4, n_group=4, topk_group=2, vocab_size=4096, quant="fp8_block",
                           num_layers=5, first_k_dense=1)
    n = 100
    ids = torch.randint(2, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(0), dtype=torch.int32).cuda()

    def run(model):
        kv = PagedKVCache(cfg, 8, 64, "cuda", torch.bfloat16)
        pages = kv.alloc.alloc(2)
        meta = AttnMeta(mode="prefill", positions=torch.arange(n, dtype=torch.int32, device="cuda"),
                        slot_mapping=torch.tensor(slots_for_range(pages, 0, n, 64), device="cuda"),
                        block_table=build_block_table([pages], "cuda"), cu_seqlens=[0, n], ctx_lens=[0])
        out = model.forward(ids, meta, kv)
        torch.cuda.synchronize()
        return out

    resident = run(build_model(cfg, "cuda", "bf16", seed=0))
    streamed = build_model(cfg, "cuda", "bf16", seed=0, stream_experts=True, ring_slots=2)
    a, b = run(streamed), run(streamed)
    _ext.check_status()
    assert torch.equal(a, resident) and torch.equal(b, resident)
    st = streamed.streamer.stats()
    assert st["modules_copied"] == 2 * 4 and st["bytes_copied"] == 2 * streamed.streamer.bytes_per_pass
    streamed.streamer.close()

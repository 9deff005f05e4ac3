"""Run under torchrun on >= 2 GPUs: ``Engine.generate`` over the fused sequence-parallel path (``forward_sp`` +
``FusedComm``), eagerly and under whole-step CUDA graphs, against the NCCL baseline engine and the unsharded
single-GPU engine on the same weights and prompts.  Rank 0 prints one JSON line."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from batchgen_b200.config import EngineConfig, get_model_config  # noqa: E402
from batchgen_b200.models import build_model  # noqa: E402
from batchgen_b200.models.weights import ParallelLayout  # noqa: E402
from batchgen_b200.ops import _ext  # noqa: E402
from batchgen_b200.parallel.comm import NcclComm  # noqa: E402
from batchgen_b200.parallel.fused import FusedComm  # noqa: E402
from batchgen_b200.runtime.engine import Engine  # noqa: E402
from batchgen_b200.runtime.graphs import DecodeGraphRunner  # noqa: E402
from batchgen_b200.runtime.sequence import SamplingParams  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = get_model_config("tiny-deepseek-v3", hidden_size=1024, q_lora_rank=512, kv_lora_rank=512,
                           qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_heads=16 * world,
                           intermediate_size=1024 * world, moe_intermediate_size=512, n_routed_experts=16,
                           num_experts_per_tok=4, n_group=4, topk_group=2, vocab_size=4096, quant="fp8_block",
                           num_layers=3, first_k_dense=1)
    g = torch.Generator().manual_seed(11)
    lens = [37, 5, 70, 129, 18, 64, 9, 200, 33, 41, 77, 3]          # sums and counts not multiples of the world size
    prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    new = 9
    sp = SamplingParams(max_new_tokens=new, ignore_eos=True)
    ecfg = lambda **kw: EngineConfig(page_size=64, max_decode_batch=16, max_prefill_tokens=256, device=str(dev),
                                     enable_cuda_graph=False, **kw)

    def run(model, graph=False, split=False, params=sp, seed=0):
        model.attn_request_parallel = split
        cfgE = ecfg(decode_attn_split="requests" if split else "heads", seed=seed)
        eng = Engine(model, cfgE, num_gpu_pages=96)
        if graph:
            eng.graph_runner = DecodeGraphRunner(model, eng.kv, max_batch=16, max_pages_per_seq=48, num_buckets=3,
                                                 max_bucket=16, sequence_parallel=eng.sp_world > 1)
        out = eng.generate(prompts, params)
        torch.cuda.synchronize()
        _ext.check_status()
        assert eng.kv.alloc.num_used == 0
        model.attn_request_parallel = False
        return out, eng

    full = build_model(cfg, dev, "bf16", seed=0)
    out_full, _ = run(full)
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    nccl_model = build_model(cfg, dev, "bf16", seed=0, layout=layout, comm=NcclComm())
    out_nccl, _ = run(nccl_model)
    comm = FusedComm(dev)
    comm.configure(cfg.hidden_size, cfg.expert_hidden, cfg.n_routed_experts, cfg.num_experts_per_tok, max_tokens=256 + 64,
                   a2a_bytes=(16 + 8 * world) * 16 * cfg.kv_cache_dim * 2)
    layout_sp = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world, sequence_parallel=True)
    sp_model = build_model(cfg, dev, "bf16", seed=0, layout=layout_sp, comm=comm)
    out_fused, eng_f = run(sp_model)
    assert eng_f.sp_world == world
    out_fused_graph, _ = run(sp_model, graph=True)
    out_fused_split, _ = run(sp_model, split=True)
    out_fused_split_graph, _ = run(sp_model, graph=True, split=True)
    # sampled decoding: every rank must hold the same tokens (uniform numbers are drawn alike on all ranks)
    samp = SamplingParams(max_new_tokens=new, ignore_eos=True, temperature=0.9, top_k=40, top_p=0.9)
    out_samp, _ = run(sp_model, params=samp, seed=5)
    flat = torch.tensor([t for o in out_samp for t in o], dtype=torch.int64, device=dev)
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    samp_consistent = bool(torch.equal(lo, hi)) and int(flat.max()) < cfg.vocab_size

    def first_agree(a, b):
        return sum(x[0] == y[0] for x, y in zip(a, b)) / len(a)

    def tok_agree(a, b):
        return sum(u == v for x, y in zip(a, b) for u, v in zip(x, y)) / sum(len(x) for x in a)

    res = {
        "world": world,
        "lengths_ok": all(len(o) == new for outs in (out_full, out_nccl, out_fused, out_fused_graph, out_fused_split,
                                                     out_fused_split_graph, out_samp) for o in outs),
        "first_fused_vs_full": first_agree(out_fused, out_full),
        "first_nccl_vs_full": first_agree(out_nccl, out_full),
        "first_fused_vs_nccl": first_agree(out_fused, out_nccl),
        "tokens_fused_vs_nccl": tok_agree(out_fused, out_nccl),
        "tokens_fused_vs_full": tok_agree(out_fused, out_full),
        "graph_equals_eager": out_fused_graph == out_fused,
        "tokens_split_vs_heads": tok_agree(out_fused_split, out_fused),
        "split_graph_equals_split": out_fused_split_graph == out_fused_split,
        "sampled_consistent": samp_consistent,
    }
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

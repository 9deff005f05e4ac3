"""Run under torchrun on >= 2 GPUs: the fused sequence-parallel forward (TP attention + EP MoE with
in-kernel NVLink communication) against the unsharded single-GPU forward of the same weights, and
against the NCCL baseline path.  Prints one JSON line per rank 0."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from batchgen_b200.config import get_model_config  # noqa: E402
from batchgen_b200.models import build_model  # noqa: E402
from batchgen_b200.models.transformer import AttnMeta  # noqa: E402
from batchgen_b200.models.weights import ParallelLayout  # noqa: E402
from batchgen_b200.ops import _ext  # noqa: E402
from batchgen_b200.parallel.comm import NcclComm  # noqa: E402
from batchgen_b200.parallel.fused import FusedComm  # noqa: E402
from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range  # noqa: E402


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
    # two sequences of different lengths; T divisible by the world size
    lens = [40 * world, 24 * world]
    if os.environ.get("BG_CHECK_LENS"):          # e.g. "384,128": rows per rank a multiple of the GEMM tile
        lens = [int(v) for v in os.environ["BG_CHECK_LENS"].split(",")]
    T = sum(lens)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(2, cfg.vocab_size, (T,), generator=g, dtype=torch.int32).to(dev)

    def meta_and_cache():
        kv = PagedKVCache(cfg, 16 + sum((n + 63) // 64 for n in lens), 64, dev, torch.bfloat16)
        pages = [kv.alloc.alloc((n + 63) // 64) for n in lens]
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(dev)
        slots = torch.tensor(sum((slots_for_range(p, 0, n, 64) for p, n in zip(pages, lens)), []), device=dev)
        cu = [0, lens[0], T]
        return AttnMeta(mode="prefill", positions=pos, slot_mapping=slots, block_table=build_block_table(pages, dev),
                        cu_seqlens=cu, ctx_lens=[0, 0]), kv

    # ---- reference: unsharded model on this GPU
    full = build_model(cfg, dev, "bf16", seed=0)
    meta, kv = meta_and_cache()
    want = full.forward(ids, meta, kv)
    Tl = T // world
    want_loc = want[rank * Tl:(rank + 1) * Tl]
    # ---- NCCL baseline: TP attention + EP MoE, replicated rows
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    nccl_model = build_model(cfg, dev, "bf16", seed=0, layout=layout, comm=NcclComm())
    meta, kv = meta_and_cache()
    got_nccl = nccl_model.forward(ids, meta, kv)[rank * Tl:(rank + 1) * Tl]
    # ---- fused sequence-parallel path
    comm = FusedComm(dev)
    comm.configure(cfg.hidden_size, cfg.expert_hidden, cfg.n_routed_experts, cfg.num_experts_per_tok, max_tokens=T,
                   a2a_bytes=T * 16 * cfg.kv_cache_dim * 2)
    # ---- chunked exchanges over peer memory against the NCCL form of the same exchange (3 rows per rank)
    xa = (torch.randn(world * 3, 192, device=dev) + rank).to(torch.bfloat16)
    got_a = comm.a2a_rows_to_ranks(xa).clone()
    want_a = NcclComm.a2a_rows_to_ranks(comm, xa)
    got_b = comm.a2a_ranks_to_rows(got_a).clone()
    want_b = NcclComm.a2a_ranks_to_rows(comm, want_a)
    a2a_ok = bool(torch.equal(got_a, want_a) and torch.equal(got_b, want_b) and got_a.shape == (3, world, 192))
    layout_sp = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world, sequence_parallel=True)
    sp_model = build_model(cfg, dev, "bf16", seed=0, layout=layout_sp, comm=comm)
    outs = []
    for _ in range(3):                       # several calls: epochs, buffer reuse
        meta, kv = meta_and_cache()
        outs.append(sp_model.forward_sp(ids, meta, kv))
    torch.cuda.synchronize()
    _ext.check_status()
    got = outs[-1]

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm())

    # ---- one decode step after the prefill, with the attention core split by request inside the TP group
    def decode_after_prefill(model, sp: bool, request_parallel: bool):
        kv = PagedKVCache(cfg, 16 + sum((n + 63) // 64 + 1 for n in lens), 64, dev, torch.bfloat16)
        pages = [kv.alloc.alloc((n + 1 + 63) // 64) for n in lens]
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(dev)
        slots = torch.tensor(sum((slots_for_range(p, 0, n, 64) for p, n in zip(pages, lens)), []), device=dev)
        bt = build_block_table(pages, dev)
        pre = AttnMeta(mode="prefill", positions=pos, slot_mapping=slots, block_table=bt, cu_seqlens=[0, lens[0], T],
                       ctx_lens=[0, 0])
        model.attn_request_parallel = False
        (model.forward_sp if sp else model.forward)(ids, pre, kv)
        nxt = torch.tensor([7, 11], dtype=torch.int32, device=dev)
        dslots = torch.tensor([slots_for_range(p, n, n + 1, 64)[0] for p, n in zip(pages, lens)], device=dev)
        dec = AttnMeta(mode="decode", positions=torch.tensor(lens, dtype=torch.int32, device=dev), slot_mapping=dslots,
                       block_table=bt, seqlens=torch.tensor([n + 1 for n in lens], dtype=torch.int32, device=dev))
        model.attn_request_parallel = request_parallel
        out = (model.forward_sp if sp else model.forward)(nxt, dec, kv)
        model.attn_request_parallel = False
        return out

    dec_rel = None
    if world == 2 and len(lens) == 2:
        d_full = decode_after_prefill(full, False, False)
        d_nccl = decode_after_prefill(nccl_model, False, True)
        d_sp = decode_after_prefill(sp_model, True, True)                  # own row only
        torch.cuda.synchronize()
        _ext.check_status()
        dec_rel = max(rel(d_nccl, d_full), rel(d_sp, d_full[rank:rank + 1]))

    res = {"rel_fused_vs_full": rel(got, want_loc), "rel_nccl_vs_full": rel(got_nccl, want_loc),
           "rel_fused_vs_nccl": rel(got, got_nccl),
           "repeatable": bool(torch.equal(outs[0], outs[-1]) and a2a_ok),
           "argmax_agree": float((got.argmax(-1) == want_loc.argmax(-1)).float().mean()),
           "nvlink_bytes": comm.nvlink_bytes, "decode_request_parallel_rel": dec_rel}
    torch.cuda.synchronize()
    dist.barrier()
    overrun = comm.heap.check_guards()        # poisoned bands after every region of the symmetric heap (BG_COMM_GUARD=1)
    t = torch.tensor([res["rel_fused_vs_full"], res["rel_nccl_vs_full"], float(res["repeatable"]),
                      res["argmax_agree"], dec_rel if dec_rel is not None else 0.0, res["rel_fused_vs_nccl"],
                      float(len(overrun))], device=dev)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tmin = t.clone()
    dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"world": world, "rel_fused_vs_full_max": float(tmax[0]), "rel_nccl_vs_full_max": float(tmax[1]),
                          "repeatable_all": bool(tmin[2] > 0.5), "argmax_agree_min": float(tmin[3]),
                          "rel_fused_vs_nccl_max": float(tmax[5]), "guard_bands_on": comm.heap.guard_bytes > 0, "nvls": bool(comm.nvls),
                          "guard_overruns_max": int(tmax[6]),
                          "nvlink_bytes": res["nvlink_bytes"],
                          "decode_request_parallel_rel_max": float(tmax[4]) if dec_rel is not None else None}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

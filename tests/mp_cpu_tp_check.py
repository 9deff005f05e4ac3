"""Child of test_multi_cpu.py: tensor-parallel attention + expert-parallel MoE over gloo (CPU, fp32) against the
unsharded model: prefill logits, one decode step with the attention core split by heads and by request."""
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
from batchgen_b200.parallel.comm import NcclComm  # noqa: E402
from batchgen_b200.runtime.kv_cache import PagedKVCache, build_block_table, slots_for_range  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = get_model_config("tiny-deepseek-v3", num_heads=4, n_routed_experts=8, num_layers=2, first_k_dense=1)
    lens = [9, 5, 12, 7]                                     # four sequences: two decode rows per rank
    T, ps = sum(lens), 16
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(2, cfg.vocab_size, (T,), generator=g, dtype=torch.int32)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)

    def run(model, request_parallel):
        kv = PagedKVCache(cfg, 32, ps, "cpu", torch.float32)
        pages = [kv.alloc.alloc((n + 1 + ps - 1) // ps) for n in lens]
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
        slots = torch.tensor(sum((slots_for_range(p, 0, n, ps) for p, n in zip(pages, lens)), []))
        bt = build_block_table(pages, "cpu")
        pre = AttnMeta(mode="prefill", positions=pos, slot_mapping=slots, block_table=bt, cu_seqlens=cu,
                       ctx_lens=[0] * len(lens))
        model.attn_request_parallel = False
        p_logits = model.forward(ids, pre, kv)
        nxt = torch.tensor([7, 11, 13, 17], dtype=torch.int32)
        dslots = torch.tensor([slots_for_range(p, n, n + 1, ps)[0] for p, n in zip(pages, lens)])
        dec = AttnMeta(mode="decode", positions=torch.tensor(lens, dtype=torch.int32), slot_mapping=dslots,
                       block_table=bt, seqlens=torch.tensor([n + 1 for n in lens], dtype=torch.int32))
        model.attn_request_parallel = request_parallel
        d_logits = model.forward(nxt, dec, kv)
        model.attn_request_parallel = False
        return p_logits, d_logits

    full = build_model(cfg, "cpu", torch.float32, seed=0)
    want_p, want_d = run(full, False)
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    comm = NcclComm()
    tp = build_model(cfg, "cpu", torch.float32, seed=0, layout=layout, comm=comm)
    got_p, got_d_heads = run(tp, False)
    _, got_d_req = run(tp, True)
    # the exchange helpers are inverses of each other and place pieces as documented
    x = torch.arange(world * 2 * 3, dtype=torch.float32).view(world * 2, 3) + 100 * rank
    y = comm.a2a_rows_to_ranks(x)                            # [2, world, 3]: piece s came from rank s
    ok_layout = all(bool(torch.equal(y[:, s], torch.arange(world * 2 * 3, dtype=torch.float32).view(world, 2, 3)[rank] + 100 * s))
                    for s in range(world))
    z = comm.a2a_ranks_to_rows(y)
    # a model with KDA layers: heads of the linear-attention layers are sharded like the MLA heads, the recurrent
    # state of a rank covers its own heads only
    kcfg = get_model_config("tiny-kimi-linear")
    klens = [6, 9]
    kids = torch.randint(2, kcfg.vocab_size, (sum(klens),), generator=g, dtype=torch.int32)

    def run_kda(model, heads):
        kv = PagedKVCache(kcfg, 16, ps, "cpu", torch.float32, state_slots=4, state_heads=heads)
        pages = [kv.alloc.alloc(1) for _ in klens]
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in klens])
        slots = torch.tensor(sum((slots_for_range(p, 0, n, ps) for p, n in zip(pages, klens)), []))
        bt = build_block_table(pages, "cpu")
        st = torch.tensor([2, 0], dtype=torch.int32)
        pre = AttnMeta(mode="prefill", positions=pos, slot_mapping=slots, block_table=bt, cu_seqlens=[0, 6, 15],
                       ctx_lens=[0, 0], state_slots=st, state_has_initial=torch.zeros(2, dtype=torch.int32))
        a = model.forward(kids, pre, kv)
        dslots = torch.tensor([slots_for_range(p, n, n + 1, ps)[0] for p, n in zip(pages, klens)])
        dec = AttnMeta(mode="decode", positions=torch.tensor(klens, dtype=torch.int32), slot_mapping=dslots,
                       block_table=bt, seqlens=torch.tensor([n + 1 for n in klens], dtype=torch.int32), state_slots=st)
        return a, model.forward(torch.tensor([5, 6], dtype=torch.int32), dec, kv)

    kfull = build_model(kcfg, "cpu", torch.float32, seed=1)
    ktp = build_model(kcfg, "cpu", torch.float32, seed=1, layout=layout, comm=comm)
    kp, kd = run_kda(kfull, kcfg.kda_num_heads)
    tp_p, tp_d = run_kda(ktp, kcfg.kda_num_heads // world)
    kda_err = max(float((tp_p - kp).abs().max()), float((tp_d - kd).abs().max()))
    # DeepSeek-V4: attention replicated on every rank, routed experts expert-parallel
    vcfg = get_model_config("tiny-deepseek-v4")
    vids = torch.randint(2, vcfg.vocab_size, (21,), generator=g, dtype=torch.int32)

    def run_v4(model):
        kv = PagedKVCache(vcfg, 8, ps, "cpu", torch.float32, state_slots=2)
        pages, slot = kv.alloc.alloc(2), kv.state.acquire()
        pre = AttnMeta(mode="prefill", positions=torch.arange(21, dtype=torch.int32),
                       slot_mapping=torch.tensor(slots_for_range(pages, 0, 21, ps)), block_table=build_block_table([pages], "cpu"),
                       cu_seqlens=[0, 21], ctx_lens=[0], state_slots=torch.tensor([slot], dtype=torch.int32))
        a = model.forward(vids, pre, kv)
        dec = AttnMeta(mode="decode", positions=torch.tensor([21], dtype=torch.int32),
                       slot_mapping=torch.tensor(slots_for_range(pages, 21, 22, ps)), block_table=build_block_table([pages], "cpu"),
                       seqlens=torch.tensor([22], dtype=torch.int32), state_slots=torch.tensor([slot], dtype=torch.int32))
        return torch.cat([a, model.forward(torch.tensor([9], dtype=torch.int32), dec, kv)])

    v_want = run_v4(build_model(vcfg, "cpu", torch.float32, seed=2))
    v_got = run_v4(build_model(vcfg, "cpu", torch.float32, seed=2, layout=layout, comm=comm))
    kda_err = max(kda_err, float((v_got - v_want).abs().max()))
    err = torch.tensor([max(float((got_p - want_p).abs().max()), kda_err), float((got_d_heads - want_d).abs().max()),
                        float((got_d_req - want_d).abs().max()), 0.0 if (ok_layout and torch.equal(z, x)) else 1.0])
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"prefill_err": float(err[0]), "decode_heads_err": float(err[1]),
                          "decode_requests_err": float(err[2]), "exchange_bad": float(err[3]),
                          "scale": float(want_p.abs().max())}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

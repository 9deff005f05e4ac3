"""Child of test_multi_cpu.py: the serving engine on two gloo ranks (TP attention + EP MoE over collectives) with
the decode attention core split by request: rows pinned to owner ranks, padded per-rank blocks, rows finishing at
different times.  Tokens must equal a single-rank engine's."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from batchgen_b200.config import EngineConfig, get_model_config  # noqa: E402
from batchgen_b200.models import build_model  # noqa: E402
from batchgen_b200.models.weights import ParallelLayout  # noqa: E402
from batchgen_b200.parallel.comm import NcclComm  # noqa: E402
from batchgen_b200.runtime.engine import Engine  # noqa: E402
from batchgen_b200.runtime.sequence import SamplingParams  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = get_model_config("tiny-deepseek-v3", num_heads=4, n_routed_experts=8)
    g = torch.Generator().manual_seed(2)
    lens = [7, 19, 11, 5, 23]                                   # five rows over two ranks: blocks of 3 and 2 (+1 pad)
    prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    news = [9, 4, 12, 6, 3]                                     # rows leave at different steps
    ecfg = EngineConfig(page_size=16, max_decode_batch=8, enable_cuda_graph=False)

    def run(model):
        eng = Engine(model, ecfg, num_gpu_pages=96)
        seqs = [eng.add_request(p, SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=True))
                for p, n in zip(prompts, news)]
        eng.run_to_completion()
        return [s.output_ids for s in seqs], [s.decode_owner for s in seqs]

    want, _ = run(build_model(cfg, "cpu", torch.float32, seed=0))
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    tp = build_model(cfg, "cpu", torch.float32, seed=0, layout=layout, comm=NcclComm())
    tp.attn_request_parallel = True
    got, owners = run(tp)
    ok = torch.tensor([1.0 if got == want else 0.0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"tokens_equal": bool(ok[0] > 0.5), "owners": owners}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

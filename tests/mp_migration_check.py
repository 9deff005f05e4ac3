"""Child of test_multi_cpu.py: a parked row moves from rank 0 to rank 1 and finishes there with the tokens an
unmoved run produces (2 gloo ranks, CPU, one rank per node)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from batchgen_b200.config import EngineConfig, get_model_config  # noqa: E402
from batchgen_b200.models import build_model  # noqa: E402
from batchgen_b200.runtime import kv_migration  # noqa: E402
from batchgen_b200.runtime.engine import Engine  # noqa: E402
from batchgen_b200.runtime.scheduler import plan_kv_migration  # noqa: E402
from batchgen_b200.runtime.sequence import S, SamplingParams  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    name = os.environ.get("BG_MIG_MODEL", "tiny-deepseek-v3")
    cfg = get_model_config(name)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(2, cfg.vocab_size, (20,), generator=g).tolist() for _ in range(3)]
    params = SamplingParams(max_new_tokens=100, temperature=0.0, ignore_eos=True)
    ecfg = EngineConfig(page_size=16, max_decode_batch=4, enable_cuda_graph=False, decision_frequency_pages=1,
                        initial_gpu_page_buffer=2, extension_gpu_page_buffer=1)

    def engine():
        return Engine(build_model(cfg, device="cpu", dtype=torch.float32, seed=0), ecfg, num_gpu_pages=64, num_host_pages=32)

    want = engine().generate(prompts, params) if rank == 0 else None
    eng = engine()
    moved_tokens = None
    if rank == 0:
        seqs = [eng.add_request(p, params) for p in prompts]
        while min(len(s.output_ids) for s in seqs) < 5:          # prefill and one decode interval
            eng.step()
        for s in seqs:
            if s.status in (S.IN_DECODE, S.PREFILLED):
                eng._hold(s)
        assert all(s.status == S.ON_HOLD and s.host_pages for s in seqs), [(s.status, len(s.output_ids)) for s in seqs]
    used = [eng.host_kv.alloc.num_used]
    allused = [None, None]
    dist.all_gather_object(allused, used[0])
    movable = [None, None]
    dist.all_gather_object(movable, [(s.global_idx, len(s.host_pages)) for s in eng.seqs.values() if s.status == S.ON_HOLD])
    plan = plan_kv_migration(allused, {0: movable[0], 1: movable[1]}, ranks_per_node=1)
    n = kv_migration.execute_plan(eng, plan, rank)
    eng.run_to_completion()
    done = {s.global_idx: s.output_ids for s in eng.seqs.values()}
    alld = [None, None]
    dist.all_gather_object(alld, done)
    if rank == 0:
        merged = {**alld[0], **alld[1]}
        ok = all(merged[i] == want[i] for i in range(len(prompts)))
        print(json.dumps({"plan": plan, "moved_here": n, "on_rank1": sorted(alld[1]), "tokens_equal": ok,
                          "host_pages_left": eng.host_kv.alloc.num_used}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

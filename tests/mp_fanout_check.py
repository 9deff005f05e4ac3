"""Two or more ranks: streamed-expert frames fanned out over NVLink into the members' ring slots (F5).
Launched by tests/test_gpu_multi.py through torch.distributed.run; prints one JSON line on rank 0."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from batchgen_b200.core import weight_replica as wr  # noqa: E402
from batchgen_b200.ops import _ext  # noqa: E402
from batchgen_b200.parallel.fanout import ReplicaFanout  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    slots, slot_bytes, layers = 3, 1 << 20, 4
    fan = ReplicaFanout(slots, slot_bytes, dev)
    ok = True
    # the replica plan decides who brings which frame: `world` experts per layer, split over the group's ranks;
    # every rank derives the same broadcast order
    group = list(range(world))
    task = {"routed_expert": [f"routed_expert_{l}_{e}" for l in range(layers) for e in range(world)]}
    fplan = wr.derive_frame_plan(task)
    owners = wr.derive_owner_map(group, task, fplan)
    order = wr.plan_broadcast_frames(task, fplan, owners)
    frames = len(order)
    g = torch.Generator().manual_seed(5)
    payloads = [torch.randint(0, 255, (slot_bytes,), dtype=torch.uint8, generator=g) for _ in range(frames)]
    for f, bf in enumerate(order):
        owner, slot = bf.owner, f % slots
        if rank == owner:
            fan.slot_view(slot).copy_(payloads[f].to(dev), non_blocking=True)     # stands in for the host -> device copy
            fan.push(slot, range(world))
        else:
            fan.wait(slot, owner)
        got = fan.slot_view(slot).clone()
        torch.cuda.synchronize()
        _ext.check_status()
        ok = ok and bool(torch.equal(got.cpu(), payloads[f]))
        dist.barrier()                                  # the slot may be reused: everybody has read this frame
    t = torch.tensor([float(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"world": world, "frames": frames, "all_equal": bool(t.item() > 0.5), "nvls": fan.nvls}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Child of test_gpu_multi.py: one rank leaves between steps; the survivors learn of it on the host before
their next launch, skip the collective, and keep a usable CUDA context.

Protocol: after every step each rank synchronises its stream and posts ``ack/<step>/<rank>`` to the control
store; before launching step k + 1 a rank waits (bounded) until every peer has either acknowledged step k or
published a down key.  The leaving rank has no kernel or collective in flight when it exits.  NCCL runs with
NVLS off and no symmetric-memory mapping exists, so no memory of the leaving rank is bound anywhere else.
"""
import datetime
import json
import os
import sys
import time

os.environ["NCCL_NVLS_ENABLE"] = "0"
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from batchgen_b200.server.restart_coordinator import RestartCoordinator, TcpStoreAdapter  # noqa: E402

LEAVE_AFTER = 3
STEPS = 6


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=20))
    store = TcpStoreAdapter("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, is_master=(rank == 0))
    coord = RestartCoordinator(rank, world, store=store, heartbeat_s=0.1, liveness_timeout_s=3.0)
    coord.beat()
    leaver = world - 1
    x = torch.ones(1 << 20, device="cuda")
    done, lost = 0, None
    for step in range(STEPS):
        if step > 0:                                   # host-side gate: every peer acked the previous step or is down
            deadline = time.monotonic() + 5.0
            while lost is None and time.monotonic() < deadline:
                lost = coord.check_peers()
                if lost is None and all(store.get(f"ack/{step - 1}/{r}") is not None for r in range(world)):
                    break
                time.sleep(0.01)
            if lost is not None:
                break
        y = x.clone()
        dist.all_reduce(y)
        torch.cuda.synchronize()
        assert float(y[0]) == world
        done += 1
        if rank == leaver and step + 1 == LEAVE_AFTER:
            coord.publish_down(0, "left between steps")        # nothing of this rank is in flight
            os._exit(0)
        coord.beat()
        store.set(f"ack/{step}/{rank}", "1")
    # survivors: the context still works, and a bounded device wait on a flag nobody sets returns a status
    a = torch.randn(256, 256, device="cuda")
    ok_math = bool(torch.isfinite(a @ a).all())
    from batchgen_b200.ops import _ext
    from batchgen_b200.parallel.fused import bounded_flag_wait
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    t0 = time.monotonic()
    bounded_flag_wait(flag, 1, epoch=1, budget_ms=200)     # the flag the lost peer would have raised
    try:
        _ext.check_status()
        status = 0
    except _ext.KernelError:
        status = 1
    waited = time.monotonic() - t0
    still_ok = bool(torch.isfinite(a @ a).all())
    if rank == 0:
        print(json.dumps({"steps_done": done, "lost": list(lost) if lost else None, "ok_math": ok_math,
                          "wait_status": int(status), "waited_s": round(waited, 3), "still_ok": still_ok}), flush=True)
    os._exit(0)          # the communicator still names the rank that left; tear nothing down collectively


if __name__ == "__main__":
    main()

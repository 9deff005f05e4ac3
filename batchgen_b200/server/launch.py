"""``python -m batchgen_b200.server.launch --model ... --world-size N``: parse flags, configure the event
log, run the fail-closed preflights, serve.  (Reference: batchgen/launch_http_server.py:35-111.)"""
from __future__ import annotations

import sys
from typing import List, Optional

from ..utils import eventlog
from .preflight import PreflightError, run_all_preflights
from .server_args import ServerArgsError, prepare_server_args


def main(argv: Optional[List[str]] = None) -> int:
    try:
        args = prepare_server_args(argv)
    except ServerArgsError as e:
        print(f"invalid flags: {e}", file=sys.stderr)
        return 2
    log = eventlog.configure_process("server", args.log_dir or None, args.log_level, console=True)
    from .server_args import REFERENCE_ACCEPTED
    for flag in getattr(args, "accepted_reference_flags", []):
        log.info("flag.accepted_without_effect", flag="--" + flag.replace("_", "-"), reason=REFERENCE_ACCEPTED[flag])
    try:
        for line in run_all_preflights(args):
            log.info("preflight", result=line)
    except PreflightError as e:
        log.error("preflight.failed", reason=str(e))
        log.close()
        return 3
    from . import run_guard
    from .runtime_lease import LaneLeaseError
    from .runtime_locks import RuntimeLockError
    try:
        guard = run_guard.acquire(args)
    except (RuntimeLockError, LaneLeaseError, ValueError) as e:
        log.error("run_guard.failed", reason=str(e))
        log.close()
        return 4
    log.info("run_guard", instance=guard.identity.instance_id, run_id=guard.identity.run_id,
             runtime_dir=str(guard.run_dir), reclaimed=guard.reclaimed, lease=guard.lease.held if guard.lease else 0)
    from .http_server import launch_server
    log.info("server.config", **{k: v for k, v in vars(args).items()})
    try:
        launch_server(args)
    except KeyboardInterrupt:
        pass
    finally:
        guard.close()
        log.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

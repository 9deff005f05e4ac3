"""Two gloo ranks on CPU: TP attention + EP MoE (collective baseline path) against the unsharded model, with
the decode attention core split by heads and by request."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_tp_ep_two_ranks_match_unsharded_model():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(HERE, "mp_cpu_tp_check.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    tol = 2e-4 * max(1.0, res["scale"])
    assert res["prefill_err"] < tol and res["decode_heads_err"] < tol and res["decode_requests_err"] < tol, res
    assert res["exchange_bad"] == 0.0, res


def _run_child(script, port, extra_env=None):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, script)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-4000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_parked_row_migrates_to_another_rank_and_finishes_there():
    res = _run_child("mp_migration_check.py", 29643)
    assert res["plan"] and res["on_rank1"], res            # the planner moved at least one row to the empty node
    assert res["tokens_equal"], res


def test_migration_carries_recurrent_state():
    res = _run_child("mp_migration_check.py", 29645, {"BG_MIG_MODEL": "tiny-kimi-linear"})
    assert res["plan"] and res["on_rank1"] and res["tokens_equal"], res


def test_engine_decodes_with_rows_pinned_to_owner_ranks():
    res = _run_child("mp_engine_split_check.py", 29647)
    assert res["tokens_equal"], res
    assert sorted(set(res["owners"])) == [0, 1], res          # both ranks own rows

"""Failure detection without any GPU fault: failures are injected on the host of gloo ranks.

* an uncaught exception on one rank ends that process at once (fail-fast hook, exit code 1) instead of
  draining collectives the peers will never complete;
* the surviving ranks' next collective ends with an error after the (short) process-group timeout, so
  nobody hangs;
* an exception in a helper thread takes the whole process down too.
"""
import os
import socket
import subprocess
import sys
import time
from pathlib import Path

WORKER = str(Path(__file__).with_name("failfast_worker.py"))


def _spawn(mode: str, world: int = 2):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), LOCAL_WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
        env.pop("PITHTRAIN_NO_FAILFAST", None)
        procs.append(subprocess.Popen([sys.executable, WORKER, mode], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    return procs


def _finish(procs, limit: float):
    t0 = time.time()
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=max(1.0, limit - (time.time() - t0)))
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\nKILLED BY TEST: still running"
        outs.append(out)
    return outs, time.time() - t0


def test_exception_on_one_rank_ends_all_ranks_quickly():
    procs = _spawn("raise")
    outs, dt = _finish(procs, 60)
    assert procs[1].returncode == 1 and "injected host-side failure" in outs[1]
    assert procs[0].returncode != 0 and "UNEXPECTED" not in outs[0] and "KILLED BY TEST" not in outs[0], outs[0][-800:]
    assert dt < 45


def test_absent_rank_times_out_the_collective():
    procs = _spawn("never_joins")
    outs, dt = _finish([procs[0]], 60)
    procs[1].kill()
    procs[1].communicate()
    assert procs[0].returncode != 0 and "UNEXPECTED" not in outs[0] and "KILLED BY TEST" not in outs[0], outs[0][-800:]


def test_exception_in_helper_thread_ends_the_process():
    procs = _spawn("thread")
    outs, dt = _finish(procs, 40)
    assert procs[0].returncode == 1 and "injected failure in a helper thread" in outs[0]
    assert dt < 25

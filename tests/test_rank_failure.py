"""Failure detection on the data-parallel path, injected on the host (no GPU, nothing faults): a rank that raises
between steps is noticed by its peer through a missed heartbeat in the rendezvous store, or through the process group's
short timeout on the next collective; either way the surviving rank returns within seconds instead of hanging."""
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "rank_failure_worker.py")


@pytest.mark.parametrize("mode,port", [("heartbeat", 29631), ("timeout", 29632)])
def test_a_failed_rank_is_detected_without_a_hang(mode, port):
    procs = []
    t0 = time.time()
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, WORKER, "--mode", mode], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()                                   # the exact process started above
            out, err = p.communicate()
            pytest.fail(f"a rank hung: {out[-1000:]} {err[-1000:]}")
        outs.append((p.returncode, out, err))
    (rc0, out0, err0), (rc1, out1, err1) = outs
    assert rc1 != 0 and "injected host-side failure" in err1
    assert "step 0 reduced" in out0 and "step 0 reduced" in out1
    assert rc0 == 0, out0[-1000:] + err0[-1000:]
    assert ("missed its heartbeat" in out0) if mode == "heartbeat" else ("ended with an error" in out0)
    assert time.time() - t0 < 90

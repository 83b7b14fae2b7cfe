"""The data-parallel contract of the path (rows sharded by rank, W replicated, one sum of dW): on CPU with gloo ranks
and the oracle, and on GPUs with NCCL, the bucketed reducer and the fused CE. Also the bucket partition arithmetic."""
import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "multi_rank_worker.py")


def _launch(backend, world, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER, "--backend", backend]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_sharded_rows_sum_to_the_full_dw_gloo():
    out = _launch("gloo", 2, 29611)
    assert "gloo world 2" in out


def test_bucket_ranges_cover_the_vocabulary():
    import nmce
    lib = nmce.Lib()
    for V, nb in ((128256, 8), (128256, 1), (1000, 8), (130, 4), (128, 3), (8257, 64)):
        v0, v1, n = (ctypes.c_int * 64)(), (ctypes.c_int * 64)(), ctypes.c_int(0)
        lib.nm_grad_bucket_ranges(V, nb, v0, v1, ctypes.byref(n))
        k = n.value
        assert 1 <= k <= nb
        assert v0[0] == 0 and v1[k - 1] == V
        for i in range(k):
            assert v0[i] % 128 == 0 and v1[i] > v0[i]
            assert v1[i] % 128 == 0 or v1[i] == V
            if i:
                assert v0[i] == v1[i - 1]
        sizes = [(v1[i] - v0[i] + 127) // 128 for i in range(k)]
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.gpu
def test_bucketed_dw_allreduce_matches_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = _launch("nccl", 2, 29612)
    assert "reduce dtype 0" in out and "reduce dtype 1" in out
    assert "zero2 rank 0" in out and "zero2 rank 1" in out      # ZeRO-2: owned accumulators of both ranks checked


@pytest.mark.gpu
def test_zero1_adamh_on_two_gpus():
    """Reduce-scatter to owners, AdamH on owned element ranges, all-gather of the bf16 replica, on 2 GPUs over NCCL,
    against the single-rank oracle (tests/adamh_rank_worker.py)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    worker = os.path.join(ROOT, "tests", "adamh_rank_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29622", worker, "--backend", "nccl"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2",
                                                                                   NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "nccl world 2" in r.stdout

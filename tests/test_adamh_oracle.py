"""The AdamH oracle (oracle/adamh_oracle.py) against what the reference's own tests pin for this update, read from
tests/s6/test_engine.cpp:723-770 (one step from mu = nu = 0 at g = 0.5: the constants 0x3DCCCCCD / 0x3CA3D70A and the
resulting mu / nu bit patterns; the Frobenius norm of p is kept to 1e-6), tests/s6/test_engine.cpp:503-534 (element
error against a host f64 reference), tests/s6/test_t1_7.py:365-369 (a zero learning rate moves p by at most 1 ulp),
docs/spec/optim.md:305-320 (table of f32 constants); and the ZeRO-1 form on two gloo ranks: per-rank partial sums over
owned element ranges, all-reduced, reproduce the single-rank update."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import adamh_oracle as A  # noqa: E402


def bits(x):
    return int(np.float32(x).view(np.uint32))


def test_constants_of_the_reference_table():
    assert bits(A.one_minus(0.9)) == 0x3DCCCCCD and bits(A.one_minus(0.98)) == 0x3CA3D70A
    assert bits(np.float32(0.9)) == 0x3F666666 and bits(np.float32(0.98)) == 0x3F7AE148
    assert bits(np.float32(A.decimal_of(1e-20))) == 0x1E3CE508 and bits(np.float32(A.decimal_of(1e-15))) == 0x26901D7D
    assert bits(A.NORM_FLOOR) == 0x2EDBE6FF
    # what a port that forms 1 - b in f32 would get instead (optim.md:311-312)
    assert bits(np.float32(1) - np.float32(0.9)) == 0x3DCCCCD0 and bits(np.float32(1) - np.float32(0.98)) == 0x3CA3D700


def test_first_step_bit_patterns_and_norm():
    rng = np.random.default_rng(1000)
    R = C = 64
    p = (rng.standard_normal((R, C)) * 0.02).astype(np.float32)
    g = np.full((R, C), 0.5, np.float32)
    z = np.zeros((R, C), np.float32)
    p2, mu, nu, _ = A.adamh_f32(p, g, z, z, 1, 0.02, 0.9, 0.98, 1e-20)
    mu_want = A.one_minus(0.9) * np.float32(0.5)
    nu_want = A.one_minus(0.98) * (np.float32(0.5) * np.float32(0.5))
    assert (mu.view(np.uint32) == bits(mu_want)).all() and (nu.view(np.uint32) == bits(nu_want)).all()
    n0, n1 = np.linalg.norm(p.astype(np.float64)), np.linalg.norm(p2.astype(np.float64))
    assert abs(n1 - n0) <= 1e-6 * n0


def _state(rng, shape):
    p = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    mu = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    nu = ((rng.standard_normal(shape) * 1e-3) ** 2).astype(np.float32)
    return p, g, mu, nu


def test_f32_order_against_f64():
    rng = np.random.default_rng(5)
    for shape, t, clip in (((96, 64), 3, False), ((33, 7), 1, True), ((257, 40), 1000, True)):
        p, g, mu, nu = _state(rng, shape)
        gn, do_clip = A.clip_state(g, 1e-3 if clip else 1e9)
        assert do_clip == clip
        p2, mu2, nu2, _ = A.adamh_f32(p, g, mu, nu, t, 0.02, 0.9, 0.98, 1e-20, clip_gn=gn, clip=do_clip, max_norm=1e-3)
        q2, m2, v2 = A.adamh_f64(p, g, mu, nu, t, 0.02, 0.9, 0.98, 1e-20, clip_gn=gn, clip=do_clip, max_norm=1e-3)
        assert np.linalg.norm(p2 - q2) <= 1e-6 * np.linalg.norm(q2)
        assert np.abs(p2 - q2).max() <= 2e-6 * np.abs(q2).max()
        assert np.abs(mu2 - m2).max() <= 1e-6 * np.abs(m2).max() and np.abs(nu2 - v2).max() <= 1e-6 * np.abs(v2).max()


def test_zero_learning_rate_moves_p_by_at_most_one_ulp():
    rng = np.random.default_rng(6)
    p, g, mu, nu = _state(rng, (64, 48))
    p2, _, _, _ = A.adamh_f32(p, g, mu, nu, 4, 0.0, 0.9, 0.98, 1e-20)
    ulp = np.abs(p2.view(np.int32).astype(np.int64) - p.view(np.int32).astype(np.int64))
    assert ulp.max() <= 1


def test_owned_ranges_tile_the_tensor():
    V, D = 1000, 16
    v0, v1 = [0, 256, 512, 768], [256, 512, 768, 1000]
    for world in (1, 2, 4, 8):
        seen = np.zeros(V * D, np.int32)
        for r in range(world):
            for off, n in A.owned_ranges(V, D, v0, v1, world, r):
                seen[off:off + n] += 1
        assert (seen == 1).all()


def test_zero1_update_on_two_gloo_ranks():
    worker = os.path.join(ROOT, "tests", "adamh_rank_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29621", worker, "--backend", "gloo"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "gloo world 2" in r.stdout

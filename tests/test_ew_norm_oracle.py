"""The numpy restatement of the levanter norm backward (oracle/ew_oracle.py) against float64 calculus: the rounding points
may only move the result by bf16 steps. CPU only."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "oracle"))
import ew_oracle  # noqa: E402

EPS = 1e-5


def _rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def _norm_bwd64(g, dy, x):
    """d/dx and d/dg of sum(dy * g * x * rsqrt(mean(x^2) + eps)) in float64."""
    D = x.shape[1]
    ms = (x * x).mean(1, keepdims=True)
    r = 1.0 / np.sqrt(ms + EPS)
    a = g[None, :] * dy
    dx = a * r - x * (r ** 3) * (x * a).sum(1, keepdims=True) / D
    dg = (dy * x * r).sum(0)
    return dx, dg, r[:, 0]


def test_bf16_rounding_is_nearest_even():
    f = np.float32
    # 1 + 2^-8 is a tie between 1 and 1 + 2^-7 (even mantissa wins); 1 + 3 * 2^-8 ties upward to 1 + 2^-6
    a = np.array([1.0, 1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, 1.0 + 2 ** -8 + 2 ** -20, -3.0e-5], f)
    got = ew_oracle.bf(a)
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == f(1.0 + 2 ** -6) and got[3] == f(1.0 + 2 ** -7)
    assert (got.view(np.uint32) & 0xFFFF == 0).all()


def test_rmsnorm_bwd_levanter_close_to_float64():
    rng = np.random.default_rng(5)
    T, D = 64, 512
    x = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 2)
    dy = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2)
    g = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    dres = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2)
    dx64, dg64, r = _norm_bwd64(g.astype(np.float64), dy.astype(np.float64), x.astype(np.float64))
    dx, gc = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, g, r.astype(np.float32), None, EPS)
    assert _rel(dx, dx64) < 6e-3 and _rel(gc.sum(0, dtype=np.float64), dg64) < 6e-3
    dx2, _ = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, g, r.astype(np.float32), dres, EPS)
    assert _rel(dx2, dx64 + dres) < 6e-3
    assert (dx.view(np.uint32) & 0xFFFF == 0).all() and (dx2.view(np.uint32) & 0xFFFF == 0).all()


def test_sandwich_bwd_levanter_close_to_float64():
    rng = np.random.default_rng(6)
    T, D = 48, 256
    xo = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32))
    b = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1.5)
    da = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2)
    dxo = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2)
    gn = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    gp = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    dxn64, dgn64, rn = _norm_bwd64(gn.astype(np.float64), da.astype(np.float64), xo.astype(np.float64))
    mid64 = dxo + dxn64
    db64, dgp64, rp = _norm_bwd64(gp.astype(np.float64), mid64, b.astype(np.float64))
    dx_in, dbr, gcn, gcp, _ = ew_oracle.sandwich_bwd_levanter(dxo, da, xo, gn, rn.astype(np.float32), b, gp,
                                                             rp.astype(np.float32), EPS)
    assert _rel(dx_in, mid64) < 8e-3 and _rel(dbr, db64) < 1.2e-2
    assert _rel(gcn.sum(0, dtype=np.float64), dgn64) < 1e-2 and _rel(gcp.sum(0, dtype=np.float64), dgp64) < 1.2e-2
    dx_in2, dbr2, _, none_p, _ = ew_oracle.sandwich_bwd_levanter(dxo, da, xo, gn, rn.astype(np.float32), None, None, None, EPS)
    assert none_p is None and np.array_equal(dx_in2, dx_in) and np.array_equal(dbr2, dx_in2)


# ----------------------------------------------------------------------------- pinned to the reference's own emulation
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "norm_golden.npz")


def _f32(bits):
    """uint16 bf16 bit patterns -> float32 values"""
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def _bits(a):
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def test_oracle_equals_reference_emulation_rmsnorm():
    """tests/golden/norm_golden.npz holds outputs of the reference's tests/s3/levemu.py (made by
    tests/golden/make_norm_golden.py): the numpy restatement must reproduce every bit."""
    G = np.load(GOLDEN)
    eps = float(G["eps"])
    for name in ("n512", "n136", "n2048"):
        x, dy, g, dres = (_f32(G[f"{name}.{k}"]) for k in ("x", "dy", "g", "dres"))
        r = G[f"{name}.rstd"]
        assert np.array_equal(_bits(ew_oracle.rmsnorm_fwd_levanter(x, g, r)), G[f"{name}.out"])
        dx, gc = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, g, r, None, eps)
        assert np.array_equal(_bits(dx), G[f"{name}.dx"]) and np.array_equal(_bits(gc), G[f"{name}.dgc"])
        dx2, _ = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, g, r, dres, eps)
        assert np.array_equal(_bits(dx2), G[f"{name}.dx_res"])


def test_oracle_equals_reference_emulation_sandwich():
    G = np.load(GOLDEN)
    eps = float(G["eps"])
    for name, post in (("s512p", True), ("s512", False), ("s136p", True), ("s2048p", True)):
        b, xi, gn, dan, dxo = (_f32(G[f"{name}.{k}"]) for k in ("b", "xi", "gn", "dan", "dxo"))
        gp = _f32(G[f"{name}.gp"]) if post else None
        rp = G[f"{name}.rp"] if post else None
        rn = G[f"{name}.rn"]
        xo, an = ew_oracle.sandwich_fwd_levanter(b, xi, gp, gn, rp, rn)
        assert np.array_equal(_bits(xo), G[f"{name}.x_out"]) and np.array_equal(_bits(an), G[f"{name}.a_next"])
        dx_in, dbr, gcn, gcp, _ = ew_oracle.sandwich_bwd_levanter(dxo, dan, xo, gn, rn, b if post else None, gp, rp, eps)
        assert np.array_equal(_bits(dx_in), G[f"{name}.dx_in"]) and np.array_equal(_bits(gcn), G[f"{name}.dgcn"])
        if post:
            # the post-norm's row sum of branch * a_post is not on a grid: torch's and numpy's float sums may differ in
            # the last bit of c, which can move a bf16 rounding of the branch gradient on a few elements by one step
            got, want = _bits(dbr).astype(np.int32), G[f"{name}.dbranch"].astype(np.int32)
            off = got != want
            assert off.mean() < 2e-3 and (np.abs(got - want)[off] <= 1).all()
            assert np.array_equal(_bits(gcp), G[f"{name}.dgcp"])
        else:
            assert np.array_equal(_bits(dbr), G[f"{name}.dx_in"])

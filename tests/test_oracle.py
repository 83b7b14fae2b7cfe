"""The CPU oracle against the golden vectors made from the reference's own Python oracles (tests/golden/make_golden.py:
tools/levref/oracle.py cross_entropy, tests/s5/nmce.py chunk_loss_ref, the grad-scale values of tests/s5/test_ce.py)."""
import numpy as np
import pytest

import ce_oracle as O


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300)


@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_numpy_oracle_matches_reference_oracle(golden, case):
    x, w, y, wt = (golden[f"{case}_{k}"] for k in ("x", "w", "labels", "weight"))
    gs = 1.0 / float(golden[f"{case}_denom"])
    loss, lse, dx, dw = O.ce_f64(x, w, y, wt, gs)
    on = wt != 0
    # the reference oracle returns the unweighted loss of every row; ours zeroes ignored rows (the kernel contract)
    assert np.abs(loss[on] - golden[f"{case}_loss"][on]).max() < 1e-12
    assert (loss[~on] == 0).all()
    assert rel(dx, golden[f"{case}_grad_x"]) < 2e-7      # golden gradients are stored as float32
    assert rel(dw, golden[f"{case}_grad_w"]) < 2e-7


@pytest.mark.parametrize("case", ["a", "b", "c"])
@pytest.mark.parametrize("f64acc", [False, True])
def test_c_oracle_matches_reference_oracle(golden, coracle, case, f64acc):
    x, w, y, wt = (golden[f"{case}_{k}"] for k in ("x", "w", "labels", "weight"))
    gs = 1.0 / float(golden[f"{case}_denom"])
    loss, lse, dx, dw = coracle.run(x, w, y, wt, gs, f64acc=f64acc)
    on = wt != 0
    assert np.abs(loss[on] - golden[f"{case}_loss"][on]).max() < 2e-5     # the reference's per-token loss bar
    assert (loss[~on] == 0).all() and (dx[~on] == 0).all()
    assert rel(dx, golden[f"{case}_grad_x"]) < 1e-5                         # the reference's f32-path bar (test_ce.py:326)
    assert rel(dw, golden[f"{case}_grad_w"]) < 1e-5


def test_chunk_loss_tree_bits(golden, coracle):
    tl, tw = golden["tree_loss"], golden["tree_weight"]
    for chunk in (1024, 2048, 4096):
        want = golden[f"tree_chunk{chunk}"]
        got_np = O.chunk_loss_tree(tl, tw, chunk)
        got_c = np.array([coracle.chunk_loss(tl[r0:r0 + chunk], tw[r0:r0 + chunk]) for r0 in range(0, tl.size, chunk)],
                         np.float32)
        assert got_np.tobytes() == want.tobytes()
        assert got_c.tobytes() == want.tobytes()


def test_grad_scale_exact_values(golden, coracle):
    for B in (128, 256):
        wt = np.ones((B, 4096), np.float32)
        wt[:, -1] = 0
        want = golden[f"grad_scale_B{B}"]
        assert O.grad_scale_tree(wt.ravel()) == want
        assert coracle.grad_scale(wt.ravel()) == want
    assert np.float32(1 / 524160) == 2 * np.float32(1 / 1048320)


def test_extensions_and_edges(coracle):
    # z-loss, an ignore index inside [0, V), label -100, weight 0, a bias: C oracle vs numpy float64
    x, w, y, wt = O.make_inputs(50, 32, 300, seed=5, ignore_frac=0.2)
    y[3] = 7
    wt[3] = 1.0
    wt[10] = 0.0
    bias = np.random.default_rng(1).standard_normal(300).astype(np.float32)
    gs = 0.01
    for zl, ii, b in ((0.0, None, None), (1e-2, 7, None), (1e-4, None, bias)):
        l64, lse64, dx64, dw64 = O.ce_f64(x, w, y, wt, gs, z_loss=zl, ignore_index=ii, bias=b)
        l, lse, dx, dw = coracle.run(x, w, y, wt, gs, z_loss=zl, ignore_index=ii, bias=b)
        assert np.abs(l - l64).max() < 2e-5 and np.abs(lse - lse64).max() < 2e-5
        assert rel(dx, dx64) < 1e-5 and rel(dw, dw64) < 1e-5
        ignored = (y < 0) | (wt == 0) | ((y == ii) if ii is not None else False)
        assert (l[ignored] == 0).all()
        assert (dx[(y < 0) | (wt == 0)] == 0).all()
    # empty input and a single row
    l, lse, dx, dw = coracle.run(x[:0], w, y[:0], wt[:0], gs)
    assert l.size == 0 and (dw == 0).all()
    l, lse, dx, dw = coracle.run(x[:1], w, y[:1], wt[:1], gs)
    l64 = O.ce_f64(x[:1], w, y[:1], wt[:1], gs)[0]
    assert np.abs(l - l64).max() < 2e-5


def test_zipf_labels():
    u = np.random.default_rng(0).random(200000)
    y = O.zipf_labels(u, 128256, 1.1)
    assert y.min() == 0 and y.max() < 128256
    c0, c1 = (y == 0).mean(), (y == 1).mean()
    assert abs(c0 / c1 - 2 ** 1.1) < 0.15


def test_doc_meta_oracle_matches_reference_numpy_reference():
    import os
    import ew_oracle as E
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ew_golden.npz"))
    got = E.doc_meta(g["dm_tok"], g["dm_valid"], int(g["dm_eos"]), int(g["dm_max_segs"]))
    want = (g["dm_targets"], g["dm_weight"], g["dm_pos"], g["dm_rss"], g["dm_cu"], int(g["dm_n"]), bool(g["dm_overflow"]))
    for name, a, b in zip(("targets", "weight", "pos", "row_seg_start", "cu_seqlens", "n", "overflow"), got, want):
        assert np.array_equal(np.asarray(a), np.asarray(b)), name
    assert bool(g["dm_overflow"]) and int(g["dm_n"]) > 6


def test_sum_fixed_oracle_is_the_chunk_loss_tree(coracle):
    import ew_oracle as E
    x = np.random.default_rng(2).standard_normal(5000).astype(np.float32)
    assert E.sum_fixed(x) == coracle.chunk_loss(x, np.ones_like(x))
    assert E.sum_fixed(np.zeros(0, np.float32)) == 0

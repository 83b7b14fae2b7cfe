"""CPU checks of the sampled-softmax head's oracle (oracle/sampled_oracle.py) and of the host arithmetic the library
shares with it: the stride of the negatives, the candidate set, and the gate the reference names for this head - the
gathered-W_P cross-entropy equals the full-vocabulary one with the logits outside the candidate set masked out
(docs/DESIGN.md:1283 of the reference)."""
import math

import numpy as np

import ce_oracle as O
import sampled_oracle as S


def test_stride_is_coprime_and_near_the_golden_ratio():
    import nmce
    lib = nmce.Lib()
    for V in (1, 2, 3, 9, 130, 1000, 8256, 64256, 128256, 1 << 20):
        s = S.sampled_stride(V)
        assert math.gcd(s, V) == 1 and 1 <= s < max(V, 2)
        if V > 100:
            assert abs(s / V - 0.6180339887) < 0.01
        assert lib.nm_ce_sampled_stride(V) == s, "the library and the oracle must walk the same negatives"
    # coprime stride: V consecutive negatives visit every id once
    V = 1000
    ids = (7 + np.arange(V) * S.sampled_stride(V)) % V
    assert np.unique(ids).size == V


def test_candidates_are_sorted_unique_targets_plus_negatives():
    rng = np.random.default_rng(1)
    V, T = 5000, 700
    y = rng.integers(0, V, T).astype(np.int32)
    y[::9] = -100
    y[5] = V + 3                          # outside the vocabulary: ignored
    wt = np.ones(T, np.float32)
    wt[::11] = 0
    cand, counts = S.candidates(y, wt, V, 300, 123456789, ignore_index=y[1])
    assert (np.diff(cand) > 0).all()
    assert set(y[counts].tolist()) <= set(cand.tolist())
    assert y[1] not in set(y[counts].tolist())
    neg = (123456789 % V + np.arange(300) * S.sampled_stride(V)) % V
    assert set(neg.tolist()) <= set(cand.tolist())
    assert cand.size <= int(counts.sum()) + 300


def test_gathered_ce_equals_masked_full_vocabulary_ce():
    x, w, y, wt = O.make_inputs(300, 64, 900, seed=4, ignore_frac=0.1)
    gs = 1.0 / float(wt.sum())
    loss, lse, dx, dw, cand = S.sampled_ce_f64(x, w, y, wt, gs, 200, 17, z_loss=1e-3)
    ml, mlse, mdx, mdw = S.masked_full_ce_f64(x, w, y, wt, gs, cand, z_loss=1e-3)
    assert np.abs(loss - ml).max() < 1e-12 and np.abs(lse - mlse).max() < 1e-12
    assert np.abs(dx - mdx).max() < 1e-14 and np.abs(dw - mdw).max() < 1e-14
    outside = np.setdiff1d(np.arange(900), cand)
    assert (dw[outside] == 0).all()

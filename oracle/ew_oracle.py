"""TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatements (numpy) of the small kernels on either side of the fused CE:
the microbatch metadata (targets / weights / positions / segment starts / packed cu_seqlens) and the fixed-order sum.
Follows wenhaochai/marin.cpp: src/kernels/elementwise/doc_meta.cu:19-81 and its numpy reference tests/s3/test_misc.py
:17-36; src/kernels/elementwise/reduce_cast.cu:93-104 (k_sum_fixed). Pinned against tests/golden/ew_golden.npz, made by
running the reference's own doc_meta_ref (tests/golden/make_golden.py)."""
import numpy as np


def doc_meta(tok, valid, eos, max_segs):
    """tok int32 [rows, S], valid bool [rows] -> (targets, weight, pos, row_seg_start [rows, max_segs + 1],
    cu_seqlens [rows * max_segs + 1], n_segments, overflow). A segment starts at position 0 and after every EOS; a row
    keeps its first max_segs starts (overflow set when it has more); unused slots hold S (rows) / rows * S (packed)."""
    tok = np.asarray(tok, np.int32)
    rows, S = tok.shape
    targets = np.concatenate([tok[:, 1:], tok[:, :1]], axis=1)
    weight = np.ones((rows, S), np.float32)
    weight[:, -1] = 0
    weight[~np.asarray(valid, bool)] = 0
    pos = np.tile(np.arange(S, dtype=np.int32), (rows, 1))
    rss = np.full((rows, max_segs + 1), S, np.int32)
    cu, overflow = [], False
    is_start = np.zeros((rows, S), bool)
    is_start[:, 0] = True
    is_start[:, 1:] = tok[:, :-1] == eos
    for r in range(rows):
        starts = np.flatnonzero(is_start[r])
        if starts.size > max_segs:
            overflow = True
            starts = starts[:max_segs]
        rss[r, :starts.size] = starts
        cu.append(r * S + starts)
    cu = np.concatenate(cu).astype(np.int32)
    cu_full = np.full(rows * max_segs + 1, rows * S, np.int32)
    cu_full[:cu.size] = cu
    return targets, weight, pos, rss, cu_full, int(cu.size), overflow


def sum_fixed(x):
    """float32 sum in the device order: 1024 thread-strided sequential sums, then a binary tree."""
    x = np.asarray(x, np.float32)
    k = (x.size + 1023) // 1024
    P = np.zeros(max(k, 1) * 1024, np.float32)
    P[:x.size] = x
    P = P.reshape(-1, 1024)
    s = np.zeros(1024, np.float32)
    for i in range(P.shape[0]):
        s = (s + P[i]).astype(np.float32)
    o = 512
    while o > 0:
        s[:o] = (s[:o] + s[o:2 * o]).astype(np.float32)
        o >>= 1
    return np.float32(s[0])

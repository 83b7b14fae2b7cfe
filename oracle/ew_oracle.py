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


# ----------------------------------------------------------------------------------------------- norm backward (levanter)
# Restates the rounding points of the reference's levanter instantiations (src/kernels/elementwise/rmsnorm_kernels.cuh:3-10,
# k_rmsnorm_bwd_add :52-100, k_sandwich_bwd :170-235): every product and sum below is one IEEE f32 operation (numpy does
# not contract), `bf` rounds to bf16 (nearest even) and widens again. Row sums are taken in float64 and rounded to f32
# once: equal to an f32 sum in ANY order whenever all partial sums are exactly representable, which the parity tests
# arrange by drawing the summed operands from small dyadic grids. The saved statistics r (rstd) are inputs, as in the
# trainer's call; rsqrtf itself is not restated. Pinned: tests/golden/norm_golden.npz holds outputs of the reference's own
# emulation of these kernels (tests/s3/levemu.py:23-44, composed as tests/s3/test_rmsnorm.py:158-176), made by
# tests/golden/make_norm_golden.py; tests/test_ew_norm_oracle.py checks this restatement against every bit of it.
def bf(a):
    """float32 array -> float32 array holding the bf16 roundings (nearest, ties to even)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(np.shape(a))


def _c2(s, r, ms, eps, n):
    f = np.float32
    return f(2) * ((s * (f(-0.5) * (r / (ms + f(eps))))) / f(n))


def _norm_bwd_rows(g, dy, x, r, eps):
    """One norm's backward over rows: returns (dx before any residual add, as bf16-valued f32; gc = bf16(dy bf16(x r));
    ms). g [D]; dy, x [T, D] bf16-valued f32; r [T] f32."""
    f = np.float32
    D = x.shape[1]
    a = bf(g[None, :] * dy)
    sxx = (x.astype(np.float64) ** 2).sum(1).astype(f)
    sxa = (x.astype(np.float64) * a.astype(np.float64)).sum(1).astype(f)
    ms = sxx / f(D)
    c2 = _c2(sxa, r, ms, eps, D)
    dx = bf(a * r[:, None] + c2[:, None] * x)
    gc = bf(dy * bf(x * r[:, None]))
    return dx, gc, ms


def rmsnorm_bwd_add_levanter(dy, x, gain, rstd, dres, eps):
    """-> (dx, gc): dx = bf16(a r + c2 x), with a residual gradient bf16(dres + dx); gc [T, D] are the per-row terms of
    the gain gradient (the kernel sums them over the rows of a part in f32)."""
    f = np.float32
    dx, gc, _ = _norm_bwd_rows(np.asarray(gain, f), np.asarray(dy, f), np.asarray(x, f), np.asarray(rstd, f), eps)
    if dres is not None:
        dx = bf(np.asarray(dres, f) + dx)
    return dx, gc


def sandwich_bwd_levanter(dx_out, da_next, x_out, g_next, rstd_next, branch, g_post, rstd_post, eps):
    """-> (dx_in, dbranch, gc_next, gc_post, sba): dx_mid = bf16(dx_out + norm_next_bwd(da_next)); dx_in = dx_mid; with a
    post-norm dbranch = norm_post_bwd(dx_mid) over the branch output, else dbranch = dx_mid. sba [T] is the post-norm's
    row sum of branch * a_post in float64 (its summands are not on a dyadic grid: callers compare dbranch with a
    tolerance of one bf16 step on a small fraction of elements)."""
    f = np.float32
    dxn, gcn, _ = _norm_bwd_rows(np.asarray(g_next, f), np.asarray(da_next, f), np.asarray(x_out, f),
                                 np.asarray(rstd_next, f), eps)
    dxm = bf(np.asarray(dx_out, f) + dxn)
    if g_post is None:
        return dxm, dxm, gcn, None, None
    b = np.asarray(branch, f)
    db, gcp, _ = _norm_bwd_rows(np.asarray(g_post, f), dxm, b, np.asarray(rstd_post, f), eps)
    ap = bf(np.asarray(g_post, f)[None, :] * dxm)
    sba = (b.astype(np.float64) * ap.astype(np.float64)).sum(1)
    return dxm, db, gcn, gcp, sba


def rmsnorm_fwd_levanter(x, gain, r):
    """out = bf16(g bf16(x r)) for given row statistics r (rmsnorm_kernels.cuh:4; the kernel's r = rsqrtf(ms + eps) is an
    approximation checked apart)."""
    f = np.float32
    return bf(np.asarray(gain, f)[None, :] * bf(np.asarray(x, f) * np.asarray(r, f)[:, None]))


def sandwich_fwd_levanter(branch, x_in, g_post, g_next, r_post, r_next):
    """-> (x_out, a_next) for given statistics: y = g_post ? bf16(g_post bf16(branch r_post)) : branch;
    x_out = bf16(x_in + y); a_next = bf16(g_next bf16(x_out r_next)) (rmsnorm_kernels.cuh:4,9, k_sandwich_fwd :100-168)."""
    f = np.float32
    b = np.asarray(branch, f)
    y = rmsnorm_fwd_levanter(b, g_post, r_post) if g_post is not None else b
    x_out = bf(np.asarray(x_in, f) + y)
    return x_out, rmsnorm_fwd_levanter(x_out, g_next, r_next)

"""CPU restatement of the reference's AdamH update of the LM head (TEST INFRASTRUCTURE ONLY: nothing in the product
imports this file; tests and the bench's CPU leg do).

What it follows in the reference:
  * operation order of the device kernels, src/kernels/optim/optk_adam.cu:1-9 (header), :19-26 (adam_dir, moments),
    :84-136 (pass 1: moments, sum p^2, sum a^2), :138-190 (w and sum w^2), :192-221 (apply), and the helpers
    src/kernels/optim/optk_common.cuh:24-30 (clip_g, norm_of: an f64 sum of f32 squares rounded to f32 once, then an
    f32 square root), :53 (sq);
  * the constants rule of docs/spec/optim.md:294-303: (1 - b) is evaluated in f64 from the decimal value of b and
    rounded to f32 once (0.9 -> 0x3DCCCCCD, 0.98 -> 0x3CA3D70A), while b * mu uses f32(b);
  * the algorithm itself, docs/spec/optim.md:264-286 (AdamH: Adam direction, then the norm-preserving projection of
    a 2-D parameter with one Frobenius norm over the whole matrix) and :123-171 (per-group clip: g <- (g / gn) * max);
  * the one-tensor entry point src/optim/capi_optim.cpp:202-219 (decimal_of, bias_correction = 1 - b^t in f32).

Two functions: adamh_f32 reproduces the f32 operation order element by element (numpy float32 arithmetic is IEEE
round-to-nearest, the same roundings as __fmul_rn / __fadd_rn / __fdiv_rn / __fsqrt_rn); adamh_f64 is the same algorithm
in float64 (the "host f64 reference" the reference's engine test compares with, tests/s6/test_engine.cpp:503-534).
"""
import numpy as np

F = np.float32
NORM_FLOOR = F(1e-10)          # docs/spec/optim.md:318 (0x2EDBE6FF)


def decimal_of(x):
    """The shortest decimal that round-trips the f32 value, as a Python float (capi_optim.cpp:61-67)."""
    return float(str(np.float32(x)))


def one_minus(b):
    """f32(1 - decimal(b)) (docs/spec/optim.md:296-303)."""
    return F(1.0 - decimal_of(b))


def bias_correction(b, t):
    """1 - f32(b)^t in f32 (capi_optim.cpp:69-72). The power is taken in f64 and rounded once; the reference uses
    XLA's f32 pow, which can differ by one ulp of b^t; AdamH divides the factor out again in its projection."""
    return F(1.0) - F(np.float64(F(b)) ** np.float64(t))


def norm_of(sumsq):
    return np.sqrt(F(sumsq))


def sumsq_f32(x):
    """f64 sum of the f32-rounded squares (optk_common.cuh:53)."""
    x = x.astype(F, copy=False)
    return float(np.sum((x * x).astype(np.float64)))


def clip_state(g, max_norm, grad_scale=1.0):
    """(gn, clip) of a clip group that holds this one tensor: gn = norm of g * grad_scale; clips unless gn < max."""
    gn = norm_of(sumsq_f32(g.astype(F) * F(grad_scale)))
    return gn, not (gn < F(max_norm))


def adamh_f32(p, g, mu, nu, t, eta, b1, b2, eps, clip_gn=0.0, clip=False, max_norm=1.0, grad_scale=1.0):
    """One AdamH step in the reference's f32 operation order. Returns (p_new, mu_new, nu_new, info)."""
    p, g, mu, nu = (np.asarray(a, dtype=F) for a in (p, g, mu, nu))
    eta, eps, max_norm, clip_gn, gs = F(eta), F(decimal_of(eps)), F(max_norm), F(clip_gn), F(grad_scale)
    fb1, fb2, omb1, omb2 = F(b1), F(b2), one_minus(b1), one_minus(b2)
    bc1, bc2 = bias_correction(b1, t), bias_correction(b2, t)
    gi = g * gs
    if clip:
        gi = (gi / clip_gn) * max_norm
    mu2 = omb1 * gi + fb1 * mu
    nu2 = omb2 * (gi * gi) + fb2 * nu
    with np.errstate(divide="ignore", invalid="ignore"):
        a = mu2 / (bc1 * (np.sqrt(nu2 / bc2) + eps))
    n = norm_of(sumsq_f32(p))
    m = norm_of(sumsq_f32(a))
    m_floor = m if (np.isnan(m) or m > NORM_FLOOR) else NORM_FLOOR
    w = p - ((eta * a) * n) / m_floor
    nw = norm_of(sumsq_f32(w))
    u = (w / nw) * n - p
    p2 = p + u
    return p2, mu2, nu2, {"n": n, "m": m, "nw": nw, "a": a}


def adam_f32(p, g, mu, nu, t, lr, b1, b2, eps, clip_gn=0.0, clip=False, max_norm=1.0, grad_scale=1.0):
    """One plain Adam step in the reference's f32 operation order (optk_adam.cu:38-82, no weight decay):
    p + ((-lr) * a). Returns (p_new, mu_new, nu_new)."""
    p, g, mu, nu = (np.asarray(a, dtype=F) for a in (p, g, mu, nu))
    lr, eps, max_norm, clip_gn, gs = F(lr), F(decimal_of(eps)), F(max_norm), F(clip_gn), F(grad_scale)
    fb1, fb2, omb1, omb2 = F(b1), F(b2), one_minus(b1), one_minus(b2)
    bc1, bc2 = bias_correction(b1, t), bias_correction(b2, t)
    gi = g * gs
    if clip:
        gi = (gi / clip_gn) * max_norm
    mu2 = omb1 * gi + fb1 * mu
    nu2 = omb2 * (gi * gi) + fb2 * nu
    with np.errstate(divide="ignore", invalid="ignore"):
        a = mu2 / (bc1 * (np.sqrt(nu2 / bc2) + eps))
    return p + (-lr) * a, mu2, nu2


def adamh_f64(p, g, mu, nu, t, eta, b1, b2, eps, clip_gn=0.0, clip=False, max_norm=1.0, grad_scale=1.0):
    """The same step in float64 from the same f32 inputs and f32 hyper-parameters."""
    p, g, mu, nu = (np.asarray(a, dtype=np.float64) for a in (p, g, mu, nu))
    eta, eps = float(F(eta)), float(F(decimal_of(eps)))
    fb1, fb2 = float(F(b1)), float(F(b2))
    omb1, omb2 = float(one_minus(b1)), float(one_minus(b2))
    bc1, bc2 = 1.0 - fb1 ** t, 1.0 - fb2 ** t
    gi = g * float(F(grad_scale))
    if clip:
        gi = (gi / float(F(clip_gn))) * float(F(max_norm))
    mu2 = omb1 * gi + fb1 * mu
    nu2 = omb2 * gi * gi + fb2 * nu
    a = mu2 / (bc1 * (np.sqrt(nu2 / bc2) + eps))
    n = np.sqrt(np.sum(p * p))
    m = max(np.sqrt(np.sum(a * a)), 1e-10)
    w = p - eta * a * n / m
    p2 = w / np.sqrt(np.sum(w * w)) * n
    return p2, mu2, nu2


def owned_ranges(V, D, v0, v1, nranks, rank):
    """Element ranges (offset, length) of the flat [V, D] tensor a rank owns when every vocabulary bucket [v0, v1) is
    split evenly, by elements, over the ranks (a reduce-scatter per bucket)."""
    out = []
    for a, b in zip(v0, v1):
        n = (b - a) * D
        assert n % nranks == 0
        out.append((a * D + rank * (n // nranks), n // nranks))
    return out


def with_row_blocks(fn, p, g, mu, nu, t, lr, b1, b2, eps, block_of_row, lr_mult=None, frozen=None, **kw):
    """A one-tensor update with a row partition (reference src/optim/capi_optim.cpp:103-128): rows of block b use the
    learning rate f32(lr * mult[b]); AdamH takes its norms over the block's rows; the rows of a frozen block keep p, mu,
    nu. fn is adamh_f32 or adam_f32 (each block is one independent call of it). Returns (p, mu, nu)."""
    p, g, mu, nu = (np.array(a, dtype=F, copy=True) for a in (p, g, mu, nu))
    block_of_row = np.asarray(block_of_row)
    for b in np.unique(block_of_row):
        if frozen is not None and frozen[b]:
            continue
        rows = block_of_row == b
        lr_b = F(F(lr) * F(1.0)) * (F(lr_mult[b]) if lr_mult is not None else F(1.0))
        out = fn(p[rows], g[rows], mu[rows], nu[rows], t, lr_b, b1, b2, eps, **kw)
        p[rows], mu[rows], nu[rows] = out[0], out[1], out[2]
    return p, mu, nu

"""TEST INFRASTRUCTURE, NOT PRODUCT CODE. The CPU oracle of the fused linear cross-entropy: a numpy float64
restatement, and a ctypes binding of the C restatement in oracle/ce_ref.c (float32, OpenMP). Only tests/, the smoke
check and bench.py's CPU-baseline legs import this module; the shipped library never does.

Follows wenhaochai/marin.cpp: the math contract include/marincpp/kernels/cross_entropy.hpp:6-15, the row kernel
src/kernels/cross_entropy/ce_logits.cu:340-384, ce_dz src/kernels/cross_entropy/ce_mma.cuh:81-85, the numpy oracle
tools/levref/oracle.py:101-127, and the fixed-order reductions ce_logits.cu:245-256 and ce_small.cu:50-61. The z-loss
term and the ignore index are extensions (z_loss = 0 and ignore_index = None reproduce the reference).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libce_ref.so")


def bf16_round(a):
    """float32 array -> float32 array holding the bf16-rounded values (round to nearest even)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(a.shape)


def ce_f64(x, w, targets, weight, grad_scale, z_loss=0.0, ignore_index=None, bias=None, tile=1024,
           want_grads=True):
    """float64 oracle. Returns (loss_tok [T], lse [T], dx [T, D] | None, dw [V, D] | None).

    loss_t = lse - z[y] + z_loss * lse^2 for a row that counts (weight != 0, 0 <= y < V, y != ignore_index), else 0;
    dz = g (p (1 + 2 z_loss lse) - onehot(y)), g = weight * grad_scale (0 for an invalid target)."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    targets = np.asarray(targets).astype(np.int64)
    weight = np.asarray(weight, np.float64)
    T, _ = x.shape
    V = w.shape[0]
    valid = (targets >= 0) & (targets < V)
    if ignore_index is not None:
        valid &= targets != ignore_index
    g_all = np.where(valid, weight * float(grad_scale), 0.0)
    loss = np.zeros(T)
    lse_all = np.zeros(T)
    dx = np.zeros_like(x) if want_grads else None
    dw = np.zeros_like(w) if want_grads else None
    for r0 in range(0, T, tile):
        r1 = min(T, r0 + tile)
        xt = x[r0:r1]
        z = xt @ w.T
        if bias is not None:
            z = z + np.asarray(bias, np.float64)[None, :]
        m = z.max(axis=1, keepdims=True)
        m = np.where(np.isfinite(m), m, 0.0)
        p = np.exp(z - m)
        s = p.sum(axis=1, keepdims=True)
        lse = (m + np.log(s))[:, 0]
        lse_all[r0:r1] = lse
        rows = np.arange(r1 - r0)
        tg = np.where(valid[r0:r1], targets[r0:r1], 0)
        counts = valid[r0:r1] & (weight[r0:r1] != 0)
        loss[r0:r1] = np.where(counts, lse - z[rows, tg] + z_loss * lse * lse, 0.0)
        if want_grads:
            p /= s
            g = g_all[r0:r1]
            p *= (g * (1.0 + 2.0 * z_loss * lse))[:, None]
            p[rows, tg] -= g
            dx[r0:r1] = p @ w
            dw += p.T @ xt
        del z, p
    return loss, lse_all, dx, dw


def chunk_loss_tree(loss, weight, chunk):
    """loss_partial[c] as the fixed-order device reduction computes it (ce_logits.cu:245-256), in float32."""
    loss = np.asarray(loss, np.float32)
    weight = np.asarray(weight, np.float32)
    out = []
    for r0 in range(0, loss.size, chunk):
        prod = (weight[r0:r0 + chunk] * loss[r0:r0 + chunk]).astype(np.float32)
        k = (prod.size + 1023) // 1024
        P = np.zeros(k * 1024, np.float32)
        P[:prod.size] = prod
        P = P.reshape(k, 1024)
        s = np.zeros(1024, np.float32)
        for i in range(k):
            s = (s + P[i]).astype(np.float32)
        o = 512
        while o > 0:
            s[:o] = (s[:o] + s[o:2 * o]).astype(np.float32)
            o >>= 1
        out.append(s[0])
    return np.array(out, np.float32)


def grad_scale_tree(weight, mult=1.0):
    """mult / sum(weight) with the fixed summation order of ce_small.cu:50-61, in float32."""
    w = np.asarray(weight, np.float32)
    k = (w.size + 1023) // 1024
    P = np.zeros(k * 1024, np.float32)
    P[:w.size] = w
    P = P.reshape(k, 1024)
    s = np.zeros(1024, np.float32)
    for i in range(k):
        s = (s + P[i]).astype(np.float32)
    o = 512
    while o > 0:
        s[:o] = (s[:o] + s[o:2 * o]).astype(np.float32)
        o >>= 1
    return np.float32(np.float32(mult) / s[0])


# ------------------------------------------------------------------------------------------------ the C oracle
def build_c(force=False):
    """Compiles oracle/ce_ref.c (make -C oracle). Returns the path of the shared object."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "ce_ref.c")):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "_build/libce_ref.so"])
    return _LIB


class COracle:
    """ctypes binding of oracle/_build/libce_ref.so."""

    def __init__(self, path=None):
        self.dll = ctypes.CDLL(path or build_c())
        P, I64, I32, F32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        for name in ("ce_ref_f32", "ce_ref_f64acc"):
            f = getattr(self.dll, name)
            f.restype = I32
            f.argtypes = [P, P, P, P, F32, P, I64, I32, I32, F32, ctypes.c_int32, I32, P, P, P, P]
        self.dll.ce_ref_chunk_loss.restype = F32
        self.dll.ce_ref_chunk_loss.argtypes = [P, P, I32]
        self.dll.ce_ref_grad_scale.restype = F32
        self.dll.ce_ref_grad_scale.argtypes = [P, I64, F32]
        self.dll.ce_ref_num_threads.restype = I32
        self.dll.ce_ref_num_threads.argtypes = []

    def threads(self):
        return int(self.dll.ce_ref_num_threads())

    def run(self, x, w, targets, weight, grad_scale, z_loss=0.0, ignore_index=None, bias=None, bf16_store=False,
            want_dx=True, want_dw=True, f64acc=False, dw_out=None):
        """float32 inputs -> (loss_tok, lse, dx | None, dw | None), all float32. dw_out: accumulate into it."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        targets = np.ascontiguousarray(targets, np.int32)
        weight = np.ascontiguousarray(weight, np.float32)
        T, D = x.shape
        V = w.shape[0]
        loss = np.zeros(T, np.float32)
        lse = np.zeros(T, np.float32)
        dx = np.zeros((T, D), np.float32) if want_dx else None
        dw = (dw_out if dw_out is not None else np.zeros((V, D), np.float32)) if want_dw else None
        b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
        ptr = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
        fn = self.dll.ce_ref_f64acc if f64acc else self.dll.ce_ref_f32
        ii = -2 ** 31 if ignore_index is None else int(ignore_index)
        rc = fn(ptr(x), ptr(w), ptr(targets), ptr(weight), float(grad_scale), ptr(b), T, D, V, float(z_loss), ii,
                int(bf16_store), ptr(loss), ptr(lse), ptr(dx), ptr(dw))
        if rc != 0:
            raise RuntimeError(f"ce_ref returned {rc}")
        return loss, lse, dx, dw

    def chunk_loss(self, loss, weight):
        loss = np.ascontiguousarray(loss, np.float32)
        weight = np.ascontiguousarray(weight, np.float32)
        return np.float32(self.dll.ce_ref_chunk_loss(loss.ctypes.data_as(ctypes.c_void_p),
                                                     weight.ctypes.data_as(ctypes.c_void_p), loss.size))

    def grad_scale(self, weight, mult=1.0):
        weight = np.ascontiguousarray(weight, np.float32)
        return np.float32(self.dll.ce_ref_grad_scale(weight.ctypes.data_as(ctypes.c_void_p), weight.size, float(mult)))


# ------------------------------------------------------------------------------------------------ synthetic inputs
def make_inputs(T, D, V, seed, ignore_frac=0.02, labels="uniform", zipf_s=1.1, w_std=0.02, bf16=True,
                ignore_index=-100):
    """Seeded synthetic inputs with the shapes and distributions of the benchmark configurations: x rows ~ N(0, 1)
    then RMS-normalised, W ~ N(0, w_std^2), both rounded to bf16 once (bf16=True) and returned as float32; labels
    uniform or Zipf(s) over [0, V) with a fraction set to ignore_index; weight = 1[label != ignore_index]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, D), dtype=np.float32)
    x /= np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)).astype(np.float32)
    w = (rng.standard_normal((V, D), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    if bf16:
        x, w = bf16_round(x), bf16_round(w)
    if labels == "uniform":
        y = rng.integers(0, V, size=T, dtype=np.int64)
    elif labels == "zipf":
        y = zipf_labels(rng.random(T), V, zipf_s)
    else:
        raise ValueError(labels)
    ign = rng.random(T) < ignore_frac
    y = np.where(ign, ignore_index, y).astype(np.int32)
    weight = (y != ignore_index).astype(np.float32)
    return x, w, y, weight


def zipf_labels(u, V, s=1.1):
    """Inverse-CDF Zipf(s) over ranks 1..V from uniforms u in [0, 1); rank 1 is id 0."""
    pk = 1.0 / np.arange(1, V + 1, dtype=np.float64) ** s
    cdf = np.cumsum(pk)
    cdf /= cdf[-1]
    return np.minimum(np.searchsorted(cdf, u, side="right"), V - 1).astype(np.int64)

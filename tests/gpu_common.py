"""Shared helpers of the GPU parity tests: the library handle, seeded inputs on the device, error metrics."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "oracle"), os.path.join(ROOT, "marin.cpp_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import ce_oracle as O  # noqa: E402  (the checker; never on the product path)
import nmce  # noqa: E402

# tolerances of the parity contract (vs the fp32 oracle on identical, already bf16-rounded inputs)
LOSS_REL = 1e-4      # scalar loss, relative
LOSS_TOK = 2e-5      # per-token loss and lse, absolute (the reference's own bar, tests/s5/test_ce.py:37)
GRAD_REL = 3e-3      # dX, dW relative L2 error
GRAD_COS = 0.9999    # dX, dW cosine

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = nmce.Lib()   # raises if the library is missing: there is no fallback
    return _lib


def rel(a, b):
    a = a.double().flatten() if torch.is_tensor(a) else torch.from_numpy(np.asarray(a, np.float64)).flatten()
    b = b.double().flatten() if torch.is_tensor(b) else torch.from_numpy(np.asarray(b, np.float64)).flatten()
    a, b = a.detach().cpu(), b.detach().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def cos(a, b):
    a = a.double().flatten().cpu() if torch.is_tensor(a) else torch.from_numpy(np.asarray(a, np.float64)).flatten()
    b = b.double().flatten().cpu() if torch.is_tensor(b) else torch.from_numpy(np.asarray(b, np.float64)).flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))


def to_dev(x, w, y, wt, dtype=torch.bfloat16):
    """numpy float32 inputs (already bf16-representable when dtype is bf16) -> device tensors"""
    return (torch.from_numpy(x).cuda().to(dtype), torch.from_numpy(w).cuda().to(dtype),
            torch.from_numpy(y).cuda().to(torch.int32), torch.from_numpy(wt).cuda().float())


def grad_scale_dev(wt):
    """1 / sum(weight) through the library's own fixed-order kernel (device scalar)"""
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    lib().nm_ce_grad_scale(nmce.ptr(wt), wt.numel(), 1.0, nmce.ptr(out), None)
    return out


def run_ce(x, W, tg, wt, gs, impl="B1", chunk=1024, fwd=False, **kw):
    V, D = W.shape
    dx = kw.pop("dx", None)
    if dx is None and not fwd:
        dx = torch.empty_like(x)
    dw = kw.pop("dw", None)
    if dw is None and not fwd:
        dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    lp = torch.empty((x.shape[0] + chunk - 1) // chunk, dtype=torch.float32, device="cuda")
    loss, lse = nmce.ce_call(lib(), impl, x, W, tg, wt, gs, dx=dx, dw=dw, loss_partial=lp, chunk=chunk,
                             forward_only=fwd, **kw)
    torch.cuda.synchronize()
    return loss, lse, dx, dw, lp


def same_bits(a, b):
    return torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))

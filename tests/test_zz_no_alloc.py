"""nm_ce_forward_noalloc, the forward-only entry point that takes no workspace and allocates nothing (its scratch is a
fixed device array inside the library), against the regular entry point run forward-only with the same chunk size.
Both launch the same kernels, so the outputs must agree to the bit, as the other forward-only checks in this suite
require. Two calls in a row on different inputs show that nothing left in the shared scratch by one call leaks into
the next. Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_forward(lib, nmce, X, W, Y, WT, chunk, z_loss, ignore_index):
    T = X.shape[0]
    lp = torch.empty((T + chunk - 1) // chunk, dtype=torch.float32, device="cuda")
    loss, lse = nmce.ce_call(lib, "B1", X, W, Y, WT, None, chunk=chunk, forward_only=True, loss_partial=lp,
                             z_loss=z_loss, ignore_index=ignore_index)
    torch.cuda.synchronize()
    return loss, lse, lp


def _noalloc_forward(lib, nmce, X, W, Y, WT, chunk, z_loss, ignore_index):
    T, D = X.shape
    V = W.shape[0]
    loss = torch.full((T,), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((T,), float("nan"), dtype=torch.float32, device="cuda")
    lp = torch.full(((T + chunk - 1) // chunk,), float("nan"), dtype=torch.float32, device="cuda")
    before = torch.cuda.memory_allocated()
    lib.nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), nmce.ptr(lse),
                              nmce.ptr(lp), T, D, V, chunk, float(z_loss), int(ignore_index), None)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return loss, lse, lp


def test_noalloc_forward_matches_workspace_forward_twice():
    from gpu_common import O, lib, nmce, same_bits, to_dev
    cases = [(3000, 512, 8256, 1024, 1e-4, -100, 21),      # several chunks, a ragged tail
             (700, 1024, 128256, 512, 0.0, 5, 22)]         # the full vocabulary; an ignore index inside [0, V)
    for T, D, V, chunk, zl, ii, seed in cases:              # two calls in a row share the built-in scratch
        x, w, y, wt = O.make_inputs(T, D, V, seed=seed, ignore_frac=0.1, labels="zipf")
        X, W, Y, WT = to_dev(x, w, y, wt)
        want = _reference_forward(lib(), nmce, X, W, Y, WT, chunk, zl, ii)
        got = _noalloc_forward(lib(), nmce, X, W, Y, WT, chunk, zl, ii)
        for name, a, b in zip(("loss_tok", "lse", "loss_partial"), got, want):
            assert same_bits(a, b), f"T{T} V{V}: {name} differs from the workspace entry point"


def test_noalloc_rejects_oversized_requests_and_accepts_nulls():
    from gpu_common import O, lib, nmce, to_dev
    x, w, y, wt = O.make_inputs(256, 64, 1000, seed=3)
    X, W, Y, WT = to_dev(x, w, y, wt)
    loss = torch.empty(256, dtype=torch.float32, device="cuda")
    with pytest.raises(nmce.NmError) as e:      # 8 * 501 * 8192 bytes > 16 MiB
        lib().nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), None, None,
                                    256, 64, 128256, 8192, 0.0, -100, None)
    assert e.value.status == 1 and "scratch" in str(e.value)
    # lse and loss_partial are optional; T == 0 is a no-op
    lib().nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), None, None, 256,
                                64, 1000, 128, 0.0, -100, None)
    torch.cuda.synchronize()
    assert torch.isfinite(loss).all()
    assert lib().nm_ce_forward_noalloc(None, None, None, None, None, None, None, 0, 64, 1000, 128, 0.0, -100, None) == 0

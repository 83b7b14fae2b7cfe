"""nm_ce_forward_noalloc, the forward-only entry point that takes no workspace and allocates nothing (its scratch is a
fixed device array inside the library), against the regular entry point run forward-only with the same chunk size.
Both launch the same kernels, so the outputs must agree to the bit, as the other forward-only checks in this suite
require. Two calls in a row on different inputs show that nothing left in the shared scratch by one call leaks into
the next. Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes
import threading

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


def _outputs(T, chunk):
    return (torch.full((T,), float("nan"), dtype=torch.float32, device="cuda"),
            torch.full((T,), float("nan"), dtype=torch.float32, device="cuda"),
            torch.full(((T + chunk - 1) // chunk,), float("nan"), dtype=torch.float32, device="cuda"))


def _noalloc_forward(lib, nmce, X, W, Y, WT, chunk, z_loss, ignore_index, stream=None):
    T, D = X.shape
    V = W.shape[0]
    loss, lse, lp = _outputs(T, chunk)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]       # the driver's count of free device bytes: sees every allocator
    lib.nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), nmce.ptr(lse),
                              nmce.ptr(lp), T, D, V, chunk, float(z_loss), int(ignore_index), stream)
    torch.cuda.synchronize()
    return (loss, lse, lp), free_before - torch.cuda.mem_get_info()[0]


def _status(lib, stream=None):
    word = ctypes.c_uint32(0xFFFF)
    lib.nm_ce_forward_noalloc_status(stream, ctypes.byref(word))
    return word.value


def test_noalloc_forward_matches_workspace_forward_twice():
    from gpu_common import O, lib, nmce, same_bits, to_dev
    cases = [(3000, 512, 8256, 1024, 1e-4, -100, 21),      # several chunks, a ragged tail
             (700, 1024, 128256, 512, 0.0, 5, 22)]         # the full vocabulary; an ignore index inside [0, V)
    for n, (T, D, V, chunk, zl, ii, seed) in enumerate(cases):   # two calls in a row share the built-in scratch
        x, w, y, wt = O.make_inputs(T, D, V, seed=seed, ignore_frac=0.1, labels="zipf")
        X, W, Y, WT = to_dev(x, w, y, wt)
        want = _reference_forward(lib(), nmce, X, W, Y, WT, chunk, zl, ii)
        got, used = _noalloc_forward(lib(), nmce, X, W, Y, WT, chunk, zl, ii)
        for name, a, b in zip(("loss_tok", "lse", "loss_partial"), got, want):
            assert same_bits(a, b), f"T{T} V{V}: {name} differs from the workspace entry point"
        assert _status(lib()) == 0
        if n > 0:   # the first call on a device may load the kernels' code; from then on not one byte may be taken
            assert used == 0, f"the call took {used} bytes of device memory"


def test_noalloc_rejects_oversized_requests_and_accepts_nulls():
    from gpu_common import O, lib, nmce, to_dev
    x, w, y, wt = O.make_inputs(256, 64, 1000, seed=3)
    X, W, Y, WT = to_dev(x, w, y, wt)
    loss = torch.empty(256, dtype=torch.float32, device="cuda")
    big_T = 8192
    with pytest.raises(nmce.NmError) as e:      # 8 * 501 * 8192 bytes > 16 MiB
        lib().nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), None, None,
                                    big_T, 64, 128256, 8192, 0.0, -100, None)
    assert e.value.status == 1 and "scratch" in str(e.value)
    # a chunk size beyond the call's rows costs nothing: 256 rows at the full vocabulary fit whatever chunk_rows says
    Wb = torch.zeros(128256, 64, dtype=torch.bfloat16, device="cuda")
    lib().nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(Wb), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), None, None, 256,
                                64, 128256, 18944, 0.0, -100, None)
    # lse and loss_partial are optional; T == 0 is a no-op
    lib().nm_ce_forward_noalloc(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss), None, None, 256,
                                64, 1000, 128, 0.0, -100, None)
    torch.cuda.synchronize()
    assert torch.isfinite(loss).all()
    assert lib().nm_ce_forward_noalloc(None, None, None, None, None, None, None, 0, 64, 1000, 128, 0.0, -100, None) == 0


def test_noalloc_status_word_can_be_read():
    """A wait that ran out inside a kernel of this entry point would leave a bit in the status word of the built-in
    scratch; nm_ce_forward_noalloc_status must report it, and the next call must start from a clean word. The bit is
    produced the safe way: the millisecond wait probe pointed at that word."""
    from gpu_common import O, lib, nmce, to_dev
    x, w, y, wt = O.make_inputs(300, 64, 500, seed=8)
    X, W, Y, WT = to_dev(x, w, y, wt)
    _noalloc_forward(lib(), nmce, X, W, Y, WT, 128, 0.0, -100)
    assert _status(lib()) == 0
    lib().nm_ce_forward_noalloc_test_timeout(1_000_000, None)
    word = ctypes.c_uint32(0)
    with pytest.raises(nmce.NmError) as e:
        lib().nm_ce_forward_noalloc_status(None, ctypes.byref(word))
    assert e.value.status == 2 and word.value == 4
    _noalloc_forward(lib(), nmce, X, W, Y, WT, 128, 0.0, -100)
    assert _status(lib()) == 0


def test_noalloc_call_from_a_thread_while_a_capture_is_open():
    """The case the entry point exists for: while one thread has a stream capture open in the global mode, no thread
    may allocate device memory. A helper thread must still be able to run a forward pass on its own stream, through
    this entry point, with buffers that existed before the capture began."""
    from gpu_common import O, lib, nmce, same_bits, to_dev
    T, D, V, chunk = 2000, 512, 8256, 1024
    x, w, y, wt = O.make_inputs(T, D, V, seed=23, ignore_frac=0.1)
    X, W, Y, WT = to_dev(x, w, y, wt)
    want = _reference_forward(lib(), nmce, X, W, Y, WT, chunk, 1e-4, -100)
    _noalloc_forward(lib(), nmce, X, W, Y, WT, chunk, 1e-4, -100)      # first use on this device: before any capture
    loss, lse, lp = _outputs(T, chunk)
    side = torch.cuda.Stream()
    cap = torch.cuda.Stream()
    static_in = torch.ones(1024, device="cuda")
    static_out = torch.empty_like(static_in)
    torch.cuda.synchronize()
    rc = []

    def helper():
        torch.cuda.set_device(0)
        rc.append(lib().raw("nm_ce_forward_noalloc")(nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(loss),
                                                     nmce.ptr(lse), nmce.ptr(lp), T, D, V, chunk, 1e-4, -100,
                                                     ctypes.c_void_p(side.cuda_stream)))

    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=cap, capture_error_mode="global"):
        torch.mul(static_in, 2.0, out=static_out)
        t = threading.Thread(target=helper)
        t.start()
        t.join()
    torch.cuda.synchronize()
    assert rc == [0], f"the call failed while a capture was open: {lib().nm_last_error()}"
    for name, a, b in zip(("loss_tok", "lse", "loss_partial"), (loss, lse, lp), want):
        assert same_bits(a, b), f"{name} differs from the workspace entry point"
    assert _status(lib()) == 0
    g.replay()
    torch.cuda.synchronize()
    assert bool((static_out == 2).all())

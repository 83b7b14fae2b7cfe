"""Parity at the configurations that are benchmarked, with the FULL dW checked: hidden 2048 / 1024 / 512 at vocabulary
128256 and the chunk size the bench runs (nm_ce_suggest_chunk_rows: 128 x SM count rows), several chunks and a 1-row
tail, against the reference's own implementation A with f32 io (its cuBLASLt true-f32 GEMMs + row kernel, what the
reference calls its reference: include/marincpp/kernels/cross_entropy.hpp:18), built unmodified into
oracle/_ref/libref_ce.so. Its f32 logits chunk for 18944 rows is 9.7 GB, which fits. Where that library was not built
the checker is the float64-accumulating CPU oracle on a row subsample plus a torch float32 chunked dW.
Also here: the reference's grid of gradient cases (tests/s5/test_ce.py:113-147), the per-layer readouts of config 4
through nm_ce_readout, the three ways the gradient contractions can get their operand, a one-rank reducer attached
to the call, and two host threads issuing calls at once.
Bars (tests/gpu_common.py): per-token loss and lse 2e-5, scalar loss 1e-4 relative, dX and dW 3e-3 relative with
cosine >= 0.9999."""
import ctypes
import os
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_ce.so")
V_FULL = 128256


class _RefLib:
    """The reference's CE module through the same ctypes signatures (it exports a subset of the entry points)."""

    def __init__(self):
        from gpu_common import nmce
        self.path = REF_LIB
        self.dll = ctypes.CDLL(REF_LIB)
        for name in ("nm_last_error", "nm_ce_workspace_bytes", "nm_fused_linear_ce"):
            f = getattr(self.dll, name)
            f.restype, f.argtypes = nmce.SIGS[name]

    def __getattr__(self, name):
        from gpu_common import nmce
        f = getattr(self.dll, name)

        def call(*a):
            r = f(*a)
            if name not in nmce.NO_STATUS and r != 0:
                raise nmce.NmError(name, r, self.dll.nm_last_error().decode())
            return r
        return call


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        return None
    return _RefLib()


def _inputs(T, D, V, labels, ignore, seed):
    """BASELINE distributions, made on the device: x rows N(0,1) RMS-normalised, W N(0, 0.02^2), both bf16; uniform or
    Zipf(1.1) labels with a fraction set to -100; weight = 1[label != -100]."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    X = torch.randn(T, D, generator=g, device="cuda")
    X = (X / X.pow(2).mean(dim=1, keepdim=True).sqrt()).to(torch.bfloat16)
    W = (torch.randn(V, D, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    if labels == "zipf":
        from gpu_common import O
        u = torch.rand(T, generator=g, device="cuda").cpu().numpy()
        Y = torch.from_numpy(O.zipf_labels(u, V, 1.1).astype(np.int32)).cuda()
    else:
        Y = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    Y[torch.rand(T, generator=g, device="cuda") < ignore] = -100
    WT = (Y != -100).float()
    return X, W, Y, WT


def _reference_a(ref, X, W, Y, WT, gs, chunk):
    """The reference's implementation A, f32 io, f32 logits store: (loss, lse, dx f32, dw f32)."""
    from gpu_common import nmce
    T, D = X.shape
    V = W.shape[0]
    Xf, Wf = X.float(), W.float()
    dx = torch.empty(T, D, dtype=torch.float32, device="cuda")
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    ws = torch.empty(ref.nm_ce_workspace_bytes(0, T, D, V, chunk, 0), dtype=torch.uint8, device="cuda")
    loss, lse = nmce.ce_call(ref, "A", Xf, Wf, Y, WT, gs, dx=dx, dw=dw, chunk=chunk, store=0, ws=ws, check=False)
    torch.cuda.synchronize()
    del ws, Xf, Wf
    return loss, lse, dx, dw


def _torch_f32(X, W, Y, WT, gs, z_loss, block=2048):
    """Fallback checker when the reference library is absent: an unfused float32 torch path, row block by row block
    (logits, softmax, dz in f32; dX and dW by f32 matmuls with TF32 off)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    T, D = X.shape
    Wf = W.float()
    dx = torch.empty(T, D, dtype=torch.float32, device="cuda")
    dw = torch.zeros_like(Wf)
    loss = torch.zeros(T, device="cuda")
    lse_all = torch.zeros(T, device="cuda")
    g = WT * gs
    for r0 in range(0, T, block):
        xb = X[r0:r0 + block].float()
        z = xb @ Wf.T
        lse = torch.logsumexp(z.double(), dim=1).float()
        lse_all[r0:r0 + block] = lse
        yb = Y[r0:r0 + block].long()
        ok = yb >= 0
        zt = z[torch.arange(z.shape[0], device="cuda"), yb.clamp_min(0)]
        loss[r0:r0 + block] = torch.where(ok, lse - zt + z_loss * lse * lse, torch.zeros_like(lse))
        p = torch.exp(z - lse[:, None]) * (g[r0:r0 + block] * (1 + 2 * z_loss * lse))[:, None]
        p[torch.arange(z.shape[0], device="cuda")[ok], yb[ok]] -= g[r0:r0 + block][ok]
        dx[r0:r0 + block] = p @ Wf
        dw += p.T @ xb
        del z, p
    return loss, lse_all, dx, dw


def rel(a, b):
    """relative L2 error, computed on the device (the tensors here are up to a gigabyte)"""
    d = (a.float() - b.float()).double().norm()
    return float(d / b.double().norm().clamp_min(1e-300))


def cos(a, b):
    a, b = a.flatten(), b.flatten()
    dot = torch.zeros((), dtype=torch.float64, device=a.device)
    for i in range(0, a.numel(), 1 << 26):           # in pieces: no full-size float64 temporaries
        dot += (a[i:i + (1 << 26)].double() * b[i:i + (1 << 26)].double()).sum()
    return float(dot / (a.double().norm() * b.double().norm()).clamp_min(1e-300))


def _compare(tag, mine, theirs, WT):
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_REL, LOSS_TOK
    loss, lse, dx, dw = mine
    rloss, rlse, rdx, rdw = theirs
    on = WT != 0
    dl = float((loss - rloss).abs().max())
    dlse = float((lse - rlse).abs().max())
    rx, cx = rel(dx, rdx), cos(dx, rdx)
    rw, cw = rel(dw, rdw), cos(dw, rdw)
    print(f"[parity] {tag}: loss {dl:.2e} lse {dlse:.2e} dX rel {rx:.2e} cos {cx:.7f} "
          f"dW rel {rw:.2e} cos {cw:.7f}")
    assert dlse <= LOSS_TOK, f"{tag}: lse {dlse:.3e}"
    assert dl <= LOSS_TOK, f"{tag}: per-token loss {dl:.3e}"
    s_m, s_r = float((loss.double() * WT).sum()), float((rloss.double() * WT).sum())
    assert abs(s_m - s_r) <= LOSS_REL * abs(s_r), f"{tag}: scalar loss {s_m} vs {s_r}"
    assert rx <= GRAD_REL and cx >= GRAD_COS, f"{tag}: dX rel {rx:.3e} cos {cx:.6f}"
    assert rw <= GRAD_REL and cw >= GRAD_COS, f"{tag}: dW rel {rw:.3e} cos {cw:.6f}"
    assert bool((loss[~on] == 0).all()) and bool((dx[~on].float() == 0).all()), f"{tag}: ignored rows must be exactly 0"


@pytest.mark.parametrize("D,chunks,labels,ignore,z_loss", [
    (2048, 2, "zipf", 0.01, 1e-4),      # config 3: two full chunks + a 1-row tail, dW += across three launches
    (1024, 1, "uniform", 0.02, 0.0),    # config 2
    (512, 1, "uniform", 0.02, 1e-4),    # configs 1 and 4 (hidden 512): the contractions form the gradient themselves
])
def test_benchmarked_shapes_with_full_dw(ref, D, chunks, labels, ignore, z_loss):
    from gpu_common import grad_scale_dev, lib, run_ce
    chunk = int(lib().nm_ce_suggest_chunk_rows(131072))
    T = chunks * chunk + 1
    X, W, Y, WT = _inputs(T, D, V_FULL, labels, ignore, seed=0xB0 + D)
    gs = grad_scale_dev(WT)
    # (i) without z-loss (the reference's API has none): everything against the reference's implementation A
    loss, lse, dx, dw, lp = run_ce(X, W, Y, WT, gs, chunk=chunk)
    if ref is not None:
        theirs = _reference_a(ref, X, W, Y, WT, gs, chunk)
        _compare(f"D{D} T{T} chunk {chunk} vs reference A/f32", (loss, lse, dx, dw), theirs, WT)
    else:
        theirs = _torch_f32(X, W, Y, WT, gs, 0.0)
        _compare(f"D{D} T{T} chunk {chunk} vs unfused f32 torch", (loss, lse, dx, dw), theirs, WT)
    del theirs
    # (ii) with the configuration's z-loss: the checker is the unfused float32 torch path, which (i) ties to the
    # reference through this library's own outputs
    if z_loss:
        del dx, dw
        loss, lse, dx, dw, lp = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=z_loss)
        theirs = _torch_f32(X, W, Y, WT, gs, z_loss)
        _compare(f"D{D} T{T} chunk {chunk} z-loss {z_loss} vs unfused f32 torch", (loss, lse, dx, dw), theirs, WT)
    assert abs(float(lp.double().sum()) - float((loss.double() * WT).sum())) <= 1e-6 * abs(float(lp.double().sum()))


@pytest.mark.parametrize("V", [512, 8256, 64256, 128256])
@pytest.mark.parametrize("D", [512, 768, 1024, 2048])
def test_reference_gradient_grid(ref, V, D):
    """The reference's own grid of gradient cases (tests/s5/test_ce.py:113-147): T = 2125 rows, every combination of
    four vocabulary and four hidden sizes. Small vocabularies go against the float64-accumulating CPU oracle, the two
    large ones against the reference's implementation A (the oracle when that library is absent)."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, O, grad_scale_dev, run_ce, to_dev
    from gpu_common import cos as cos_np, rel as rel_np
    T = 2125
    x, w, y, wt = O.make_inputs(T, D, V, seed=V + D, ignore_frac=0.03)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    loss, lse, dx, dw, _ = run_ce(X, W, Y, WT, gs, chunk=1024)
    if V >= 64256 and ref is not None:
        _compare(f"grid V{V} D{D} vs reference A/f32", (loss, lse, dx, dw), _reference_a(ref, X, W, Y, WT, gs, 1024), WT)
        return
    if not hasattr(test_reference_gradient_grid, "oracle"):
        test_reference_gradient_grid.oracle = O.COracle()
    ol, olse, odx, odw = test_reference_gradient_grid.oracle.run(x, w, y, wt, float(gs.item()), f64acc=True)
    rx, rw = rel_np(dx, odx), rel_np(dw, odw)
    print(f"[parity] grid V{V} D{D} vs oracle: loss {np.abs(loss.cpu().numpy() - ol).max():.2e} dX rel {rx:.2e} dW rel {rw:.2e}")
    assert np.abs(loss.cpu().numpy() - ol).max() <= LOSS_TOK and np.abs(lse.cpu().numpy() - olse).max() <= LOSS_TOK
    assert rx <= GRAD_REL and cos_np(dx, odx) >= GRAD_COS and rw <= GRAD_REL and cos_np(dw, odw) >= GRAD_COS


def test_three_gradient_paths_agree():
    """The in-place pass + 128 x 256 tiles, the pass + 256 x 512 pair tiles, and the pair tiles that form the gradient in
    shared memory compute the same thing: loss, lse and dX bit for bit (each dX element is the same sum in the same
    order), dW up to the order in which tiles of different shape add their K blocks (it is the same order here too,
    so bit-equality is asserted where the row count per chunk is the same)."""
    from gpu_common import O, grad_scale_dev, lib, run_ce, same_bits, to_dev
    for T, D, V, chunk in ((3000, 512, 8256, 1024), (1500, 1024, 16400, 1500), (700, 2048, 1000, 512),
                           (2100, 264, 8257, 1022)):
        x, w, y, wt = O.make_inputs(T, D, V, seed=T + D, ignore_frac=0.05, labels="zipf")
        X, W, Y, WT = to_dev(x, w, y, wt)
        gs = grad_scale_dev(WT)
        outs = []
        try:
            for path in (0, 1, 2):
                lib().nm_ce_set_grad_path(path)
                outs.append(run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4))
        finally:
            lib().nm_ce_set_grad_path(-1)
        for path in (1, 2):
            for i, name in enumerate(("loss", "lse", "dx", "dw", "loss_partial")):
                assert same_bits(outs[path][i], outs[0][i]), f"T{T} D{D} V{V}: path {path} vs 0: {name} differs"


def test_readouts_accumulate_into_one_dw(ref):
    """Config 4's shape through nm_ce_readout: three per-layer readouts (independent states, shared head and labels)
    accumulate into one dW. Checker: the normed activations this library produced (bf16) go through the reference's
    implementation A one readout at a time; its dW summed over the readouts, and its dX pushed through a float64 torch
    RMSNorm backward, are what dW and d_state must match."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, grad_scale_dev, lib, nmce
    T, D, V, R = 16384, 512, V_FULL, 3
    chunk = int(lib().nm_ce_suggest_chunk_rows(T))
    _, W, Y, WT = _inputs(T, D, V, "uniform", 0.02, seed=0xC4)
    gs = grad_scale_dev(WT) / R
    g = torch.Generator(device="cuda").manual_seed(44)
    gain = (1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")).to(torch.bfloat16)
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    want_dw = torch.zeros_like(dw)
    ws = torch.empty(lib().nm_ce_workspace_bytes(1, T, D, V, chunk, 1), dtype=torch.uint8, device="cuda")
    P = int(lib().nm_norm_partial_rows(T))
    for layer in range(R):
        S = (torch.randn(T, D, generator=g, device="cuda") * (1.0 + layer)).to(torch.bfloat16)
        normed = torch.empty_like(S)
        normed_copy = torch.empty_like(S)
        rstd = torch.empty(T, device="cuda")
        d_state = torch.zeros_like(S)
        part = torch.zeros(P, D, device="cuda")
        loss = torch.empty(T, device="cuda")
        lse = torch.empty(T, device="cuda")
        lp = torch.empty((T + chunk - 1) // chunk, device="cuda")
        lib().nm_rmsnorm_fwd(1, 1, nmce.ptr(S), nmce.ptr(gain), nmce.ptr(normed_copy), nmce.ptr(rstd), T, D, 1e-5, None)
        lib().nm_ce_readout(1, 1, 1, nmce.ptr(S), nmce.ptr(gain), nmce.ptr(rstd), nmce.ptr(normed), nmce.ptr(W),
                            nmce.ptr(dw), nmce.ptr(part), nmce.ptr(gs), nmce.ptr(d_state), D, nmce.ptr(Y), nmce.ptr(WT),
                            nmce.ptr(loss), nmce.ptr(lse), nmce.ptr(lp), 0, T, D, V, chunk, 1e-5, nmce.ptr(ws), None)
        st = ctypes.c_uint32(0)
        lib().nm_ce_device_status(nmce.ptr(ws), None, ctypes.byref(st))
        if ref is not None:
            rl, rlse, rdx, rdw = _reference_a(ref, normed_copy, W, Y, WT, gs, chunk)
        else:
            rl, rlse, rdx, rdw = _torch_f32(normed_copy, W, Y, WT, gs, 0.0)
        want_dw += rdw
        assert float((loss - rl).abs().max()) <= LOSS_TOK and float((lse - rlse).abs().max()) <= LOSS_TOK
        # the norm's backward in float64 on the checker's dX (accurate rounding: one rounding of the stored output)
        s64 = S.double().requires_grad_(True)
        y64 = s64 * torch.rsqrt(s64.pow(2).mean(dim=1, keepdim=True) + 1e-5) * gain.double()
        y64.backward(rdx.double())
        rs = rel(d_state, s64.grad)
        print(f"[parity] readout {layer}: d_state rel {rs:.2e}")
        assert rs <= GRAD_REL and cos(d_state, s64.grad) >= GRAD_COS
        del s64, y64
    rw, cw = rel(dw, want_dw), cos(dw, want_dw)
    print(f"[parity] {R} readouts of {T} x {D}: accumulated dW rel {rw:.2e} cos {cw:.7f}")
    assert rw <= GRAD_REL and cw >= GRAD_COS


def test_one_rank_reducer_attached_to_the_call():
    """A communicator of ONE rank and a bucketed reducer attached to the call: the last chunk's dW then runs bucket by
    bucket with SMs set aside for the collective, each bucket is 'reduced' (over one rank: the identity) on the
    communication stream, and dX runs beside it. In f32 the result must be the plain call's bits; with the bf16 wire
    format every element passes through bf16 exactly once, so it must equal the plain dW rounded to bf16."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, same_bits, to_dev
    T, D, V, chunk = 4500, 1024, 16400, 2048
    x, w, y, wt = O.make_inputs(T, D, V, seed=91, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    plain = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4)
    idbuf = torch.zeros(128, dtype=torch.uint8)
    lib().nm_comm_unique_id(nmce.ptr(idbuf))
    comm = ctypes.c_void_p()
    lib().nm_comm_create(nmce.ptr(idbuf), 1, 0, ctypes.byref(comm))
    try:
        for reduce_dtype in (0, 1):
            dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
            staging = torch.empty(V, D, dtype=torch.bfloat16, device="cuda") if reduce_dtype else None
            red = ctypes.c_void_p()
            lib().nm_grad_reducer_create(comm, nmce.ptr(dw), V, D, 5, reduce_dtype, nmce.ptr(staging), ctypes.byref(red))
            try:
                got = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4, dw=dw, reducer=red)
                lib().nm_grad_reducer_wait(red, None)
                torch.cuda.synchronize()
            finally:
                lib().nm_grad_reducer_destroy(red)
            for i, name in enumerate(("loss", "lse", "dx")):
                assert same_bits(got[i], plain[i]), f"reduce dtype {reduce_dtype}: {name} differs from the plain call"
            want = plain[3] if reduce_dtype == 0 else plain[3].to(torch.bfloat16).float()
            assert same_bits(dw, want), f"reduce dtype {reduce_dtype}: dW differs"
        # dX written over x keeps the dW-first order of the last chunk; the other order (dX first) ran above
        dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
        red = ctypes.c_void_p()
        lib().nm_grad_reducer_create(comm, nmce.ptr(dw), V, D, 5, 0, None, ctypes.byref(red))
        try:
            xi = X.clone()
            run_ce(xi, W, Y, WT, gs, chunk=chunk, z_loss=1e-4, dx=xi, dw=dw, reducer=red)
            lib().nm_grad_reducer_wait(red, None)
            torch.cuda.synchronize()
        finally:
            lib().nm_grad_reducer_destroy(red)
        assert same_bits(xi, plain[2]) and same_bits(dw, plain[3]), "dx == x with a reducer differs from the plain call"
    finally:
        lib().nm_comm_destroy(comm)


def test_one_rank_zero2_accumulates_owned_slices():
    """ZeRO-2 for the head gradient on a communicator of one rank (reduce-scatter over one rank: the identity): an owners
    reducer attached to every microbatch, nm_grad_reducer_microbatch_done after each. The packed accumulator must hold
    the sum of the microbatches' dW (bit for bit here: every microbatch is one chunk, so each element receives the same
    additions in the same order as in a plain call that accumulates all microbatches into one buffer), the [V, D]
    buffer must be zero afterwards, and nm_grad_reducer_owned_to_grad must put the sums back where an optimizer on
    owned elements reads them."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, same_bits, to_dev
    D, V, chunk, micro = 512, 8256, 2048, 3
    rows = [1500, 2048, 700]
    idbuf = torch.zeros(128, dtype=torch.uint8)
    lib().nm_comm_unique_id(nmce.ptr(idbuf))
    comm = ctypes.c_void_p()
    lib().nm_comm_create(nmce.ptr(idbuf), 1, 0, ctypes.byref(comm))
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    plain_dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    red = ctypes.c_void_p()
    lib().nm_grad_reducer_create_owners(comm, nmce.ptr(dw), V, D, 5, ctypes.byref(red))
    try:
        n_owned = int(lib().nm_grad_reducer_owned_elems(red))
        assert n_owned == V * D
        acc = torch.zeros(n_owned, dtype=torch.float32, device="cuda")
        for m in range(micro):
            x, w, y, wt = O.make_inputs(rows[m], D, V, seed=300 + m, ignore_frac=0.05)
            if m:
                w = w0
            w0 = w
            X, W, Y, WT = to_dev(x, w, y, wt)
            gs = grad_scale_dev(WT)
            run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4, dw=plain_dw)            # accumulates across microbatches
            run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4, dw=dw, reducer=red)
            lib().nm_grad_reducer_microbatch_done(red, nmce.ptr(acc), None)
            torch.cuda.synchronize()
            assert not dw.any(), "the gradient buffer must be zero after microbatch_done"
        assert same_bits(acc.view(V, D), plain_dw)
        lib().nm_grad_reducer_owned_to_grad(red, nmce.ptr(acc), None)
        torch.cuda.synchronize()
        assert same_bits(dw, plain_dw)
    finally:
        lib().nm_grad_reducer_destroy(red)
        lib().nm_comm_destroy(comm)


def test_two_host_threads_call_concurrently():
    """Two host threads, each with its own stream, workspace and outputs, issue the same call on one GPU at the same
    time (the reference's trainer enters the library from one thread per GPU, src/train/trainer.cpp:57,209-219; here the
    threads share a device so that the test runs on one GPU). Every result must carry the bits of the serial call."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, same_bits, to_dev
    T, D, V, chunk = 3000, 512, 8256, 1024
    x, w, y, wt = O.make_inputs(T, D, V, seed=13, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    serial = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4)
    nb = lib().nm_ce_workspace_bytes(1, T, D, V, chunk, 1)
    results, errors = {}, []
    barrier = threading.Barrier(2)

    def worker(i):
        try:
            torch.cuda.set_device(0)
            s = torch.cuda.Stream()
            ws = torch.empty(nb, dtype=torch.uint8, device="cuda")
            outs = []
            barrier.wait()
            for _ in range(6):
                dx = torch.empty_like(X)
                dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
                lp = torch.empty((T + chunk - 1) // chunk, dtype=torch.float32, device="cuda")
                with torch.cuda.stream(s):
                    dw.zero_()
                    loss, lse = nmce.ce_call(lib(), "B1", X, W, Y, WT, gs, dx=dx, dw=dw, loss_partial=lp, chunk=chunk,
                                             ws=ws, z_loss=1e-4, stream=s.cuda_stream, check=False)
                    lib().nm_ce_set_backends(i, i, -1)          # the process-wide switches are touched meanwhile
                    lib().nm_ce_suggest_chunk_rows(T)
                outs.append((loss, lse, dx, dw, lp))
            s.synchronize()
            st = ctypes.c_uint32(0)
            lib().nm_ce_device_status(nmce.ptr(ws), ctypes.c_void_p(s.cuda_stream), ctypes.byref(st))
            results[i] = outs
        except Exception as e:   # noqa: BLE001 (reported below, in the main thread)
            errors.append(e)
            try:
                barrier.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    lib().nm_ce_set_backends(0, 0, -1)
    assert not errors, errors
    torch.cuda.synchronize()
    for i in range(2):
        for outs in results[i]:
            for k, name in enumerate(("loss", "lse", "dx", "dw", "loss_partial")):
                assert same_bits(outs[k], serial[k]), f"thread {i}: {name} differs from the serial call"


def test_thread_per_gpu():
    """The reference's own threading form: one host thread per GPU, all inside the call at once; same bits on every GPU."""
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    from gpu_common import O, lib, nmce, same_bits
    T, D, V, chunk = 2500, 768, 8256, 1024
    x, w, y, wt = O.make_inputs(T, D, V, seed=14, ignore_frac=0.05)
    results, errors = {}, []
    barrier = threading.Barrier(n)

    def worker(dev):
        try:
            torch.cuda.set_device(dev)
            d = torch.device("cuda", dev)
            X = torch.from_numpy(x).to(d).bfloat16()
            W = torch.from_numpy(w).to(d).bfloat16()
            Y = torch.from_numpy(y).to(d)
            WT = torch.from_numpy(wt).to(d)
            gs = torch.empty(1, dtype=torch.float32, device=d)
            lib().nm_ce_grad_scale(nmce.ptr(WT), T, 1.0, nmce.ptr(gs), None)
            ws = torch.empty(lib().nm_ce_workspace_bytes(1, T, D, V, chunk, 1), dtype=torch.uint8, device=d)
            dx = torch.empty_like(X)
            dw = torch.zeros(V, D, dtype=torch.float32, device=d)
            barrier.wait()
            loss, lse = nmce.ce_call(lib(), "B1", X, W, Y, WT, gs, dx=dx, dw=dw, chunk=chunk, ws=ws)
            torch.cuda.synchronize(d)
            results[dev] = [t.cpu() for t in (loss, lse, dx, dw)]
        except Exception as e:   # noqa: BLE001
            errors.append(e)
            try:
                barrier.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=worker, args=(d,)) for d in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for dev in range(1, n):
        for a, b in zip(results[0], results[dev]):
            assert same_bits(a, b)

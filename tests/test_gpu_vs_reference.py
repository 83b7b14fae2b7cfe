"""Parity against the REFERENCE ITSELF: the reference's fused-CE module, compiled unmodified for sm_100a by
oracle/Makefile (target _ref/libref_ce.so), driven through the same C ABI and the same ctypes harness as this library.
Its implementation A with f32 io (true-f32 cuBLASLt GEMMs + a row kernel) is what the reference calls its reference
(include/marincpp/kernels/cross_entropy.hpp:18) and what its kernel tests compare against; its B1 is what it would run
in training on a B200 (portable mma.sync logits kernel + cuBLASLt). Skipped when the library was not built."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_ce.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libref_ce.so was not built (make -C oracle _ref/libref_ce.so)")
    from gpu_common import nmce
    import ctypes
    dll = ctypes.CDLL(REF_LIB)

    class RefLib:     # the reference exports a subset of the entry points: bind only those
        path = REF_LIB

        def __init__(self):
            self.dll = dll
            for name in ("nm_last_error", "nm_ce_workspace_bytes", "nm_fused_linear_ce", "nm_ce_grad_scale",
                         "nm_ce_set_backends"):
                f = getattr(dll, name)
                f.restype, f.argtypes = nmce.SIGS[name]

        def __getattr__(self, name):
            f = getattr(dll, name)

            def call(*a):
                r = f(*a)
                if name not in nmce.NO_STATUS and r != 0:
                    raise nmce.NmError(name, r, dll.nm_last_error().decode())
                return r
            return call
    return RefLib()


def _ref_call(ref, impl, X, W, Y, WT, gs, chunk, store=1):
    from gpu_common import nmce
    T, D = X.shape
    V = W.shape[0]
    dx = torch.empty_like(X)
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    lp = torch.empty((T + chunk - 1) // chunk, dtype=torch.float32, device="cuda")
    ws = torch.empty(ref.nm_ce_workspace_bytes(nmce.IMPLS[impl], T, D, V, chunk, store), dtype=torch.uint8, device="cuda")
    loss, lse = nmce.ce_call(ref, impl, X, W, Y, WT, gs, dx=dx, dw=dw, loss_partial=lp, chunk=chunk, store=store, ws=ws,
                             check=False)
    torch.cuda.synchronize()
    return loss, lse, dx, dw, lp


@pytest.mark.parametrize("T,D,V,labels", [(2125, 512, 8256, "uniform"), (1500, 2048, 16384, "zipf"),
                                          (700, 1024, 128256, "uniform")])
def test_against_the_reference_f32_implementation(ref, T, D, V, labels):
    """This library (bf16 io) against the reference's implementation A with f32 io on the same (bf16-representable)
    inputs: the north-star parity statement. Bars: scalar loss 1e-4 relative, per-token 2e-5, dX / dW 3e-3, cos 0.9999."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_REL, LOSS_TOK, O, cos, grad_scale_dev, rel, run_ce, to_dev
    x, w, y, wt = O.make_inputs(T, D, V, seed=T + V, ignore_frac=0.02, labels=labels)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    mine = run_ce(X, W, Y, WT, gs, chunk=1024)
    theirs = _ref_call(ref, "A", X.float(), W.float(), Y, WT, gs, 1024, store=0)
    on = (WT != 0)
    dl = float((mine[0] - theirs[0]).abs().max())
    dlse = float((mine[1] - theirs[1]).abs().max())
    s_m = float((mine[0].double() * WT).sum())
    s_t = float((theirs[0].double() * WT).sum())
    rx, cx = rel(mine[2], theirs[2]), cos(mine[2], theirs[2])
    rw, cw = rel(mine[3], theirs[3]), cos(mine[3], theirs[3])
    print(f"[parity] vs reference A/f32 T{T} D{D} V{V}: loss {dl:.2e} lse {dlse:.2e} dX rel {rx:.2e} cos {cx:.7f} "
          f"dW rel {rw:.2e} cos {cw:.7f}")
    assert dl <= LOSS_TOK and dlse <= LOSS_TOK
    assert abs(s_m - s_t) <= LOSS_REL * abs(s_t)
    assert rx <= GRAD_REL and cx >= GRAD_COS and rw <= GRAD_REL and cw >= GRAD_COS
    assert bool((mine[0][~on] == 0).all()) and bool((theirs[0][~on] == 0).all())


def test_against_the_reference_training_path_and_shared_bits(ref):
    """The reference's B1 (what its trainer runs) on the same bf16 inputs; and the pieces that are specified to the bit:
    the grad scale and, given the same per-token losses, the per-chunk loss tree."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, O, cos, grad_scale_dev, lib, nmce, rel, run_ce, to_dev
    T, D, V, chunk = 3000, 768, 8256, 1024
    x, w, y, wt = O.make_inputs(T, D, V, seed=5, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    gs_ref = torch.empty(1, dtype=torch.float32, device="cuda")
    ref.nm_ce_grad_scale(nmce.ptr(WT), T, 1.0, nmce.ptr(gs_ref), None)
    torch.cuda.synchronize()
    assert gs.item() == gs_ref.item(), "grad scale bits differ from the reference's kernel"
    mine = run_ce(X, W, Y, WT, gs, chunk=chunk)
    for own in (0, 1):
        ref.nm_ce_set_backends(own, own, -1)
        theirs = _ref_call(ref, "B1", X, W, Y, WT, gs, chunk)
        assert float((mine[0] - theirs[0]).abs().max()) <= LOSS_TOK
        assert float((mine[1] - theirs[1]).abs().max()) <= LOSS_TOK
        rx, rw = rel(mine[2], theirs[2]), rel(mine[3], theirs[3])
        print(f"[parity] vs reference B1 ({'own' if own else 'cuBLASLt'} GEMMs): dX rel {rx:.2e} dW rel {rw:.2e}")
        # both are bf16-rounded results of the same quantity: each is within 1.7e-3 of the truth
        assert rx <= 1.5 * GRAD_REL and rw <= 1.5 * GRAD_REL
        assert cos(mine[2], theirs[2]) >= GRAD_COS and cos(mine[3], theirs[3]) >= GRAD_COS
    ref.nm_ce_set_backends(0, 0, -1)
    want = O.chunk_loss_tree(theirs[0].cpu().numpy(), wt, chunk)
    assert theirs[4].cpu().numpy().tobytes() == want.tobytes(), "the oracle's loss tree is the reference kernel's, to the bit"


# ------------------------------------------------------------------------------------------------ AdamH of the head
REF_OPT = os.path.join(ROOT, "oracle", "_ref", "libref_optim.so")


@pytest.mark.parametrize("shape,t,clip", [((2048, 512), 1, False), ((1000, 264), 7, True), ((8192, 2048), 300, True)])
def test_adamh_update_against_the_reference_library(shape, t, clip):
    """nm_adamh_update of this library against the reference's own implementation of the same entry point
    (src/optim/capi_optim.cpp:202-219 -> engine -> optk_adam.cu), built unmodified for sm_100a. Moments must be
    bit-equal (element arithmetic in the same order); the parameters agree to 1e-6, the bar the reference holds between
    its own scalar and float4 paths, whose norms sum in different orders (tests/s6/test_engine.cpp:538-590)."""
    if not os.path.exists(REF_OPT):
        pytest.skip("oracle/_ref/libref_optim.so was not built (make -C oracle _ref/libref_optim.so)")
    import ctypes
    import time
    from gpu_common import lib, nmce
    rdll = ctypes.CDLL(REF_OPT)
    rdll.nm_adamh_update.restype, rdll.nm_adamh_update.argtypes = nmce.SIGS["nm_adamh_update"]
    rdll.nm_last_error.restype = ctypes.c_char_p
    rng = np.random.default_rng(shape[0] + t)
    p = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    mu = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    nu = ((rng.standard_normal(shape) * 1e-3) ** 2).astype(np.float32)
    gn = float(np.sqrt(np.float32(np.sum((g * g).astype(np.float64)))))
    max_norm = 0.5 * gn if clip else 1.0
    out = {}
    for name, fn in (("ours", lib().raw("nm_adamh_update")), ("ref", rdll.nm_adamh_update)):
        P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
        P16 = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rc = fn(nmce.ptr(P), nmce.ptr(P16), nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), shape[0], shape[1], t, 0.02, 0.9,
                0.98, 1e-20, gn, int(clip), max_norm, None, None, None, 0, None)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        assert rc == 0, (name, rdll.nm_last_error())
        out[name] = (P, M, V, P16, ms)
    (P, M, V, P16, ms), (RP, RM, RV, RP16, rms) = out["ours"], out["ref"]
    assert torch.equal(M, RM) and torch.equal(V, RV), "moments differ from the reference's bits"
    r = float((P.double() - RP.double()).norm() / RP.double().norm())
    assert r <= 1e-6, f"p rel {r:.3e}"
    assert int((P16 != RP16).sum()) <= 1e-4 * P16.numel()       # an f32 difference of 1 ulp can flip a bf16 tie
    print(f"AdamH {shape} t={t}: p rel vs reference {r:.2e}; host wall of one call {ms:.2f} ms vs reference {rms:.2f} ms")


def test_adam_update_against_the_reference_library():
    """nm_adam_update against the reference's (src/optim/capi_optim.cpp:221-238): bit-equal at t = 1 (bias corrections
    1 - b exactly); at other t the reference's table uses XLA's f32 pow, this library a correctly rounded one, which may
    differ by an ulp of b^t: the parameters then agree to 1e-7."""
    if not os.path.exists(REF_OPT):
        pytest.skip("oracle/_ref/libref_optim.so was not built (make -C oracle _ref/libref_optim.so)")
    import ctypes
    from gpu_common import lib, nmce
    rdll = ctypes.CDLL(REF_OPT)
    rdll.nm_adam_update.restype, rdll.nm_adam_update.argtypes = nmce.SIGS["nm_adam_update"]
    rng = np.random.default_rng(3)
    shape = (64, 2048)
    p = (rng.standard_normal(shape) * 0.5 + 1.0).astype(np.float32)
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    mu = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    nu = ((rng.standard_normal(shape) * 1e-3) ** 2).astype(np.float32)
    for t in (1, 25, 1000):
        out = []
        for fn in (lib().raw("nm_adam_update"), rdll.nm_adam_update):
            P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
            assert fn(nmce.ptr(P), None, nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), shape[0], shape[1], t, 0.008, 0.9, 0.98,
                      1e-20, 0.0, 0, 1.0, None, None, None, 0, None) == 0
            torch.cuda.synchronize()
            out.append((P, M, V))
        (P, M, V), (RP, RM, RV) = out
        assert torch.equal(M, RM) and torch.equal(V, RV)
        if t == 1:
            assert torch.equal(P, RP)
        else:
            assert float((P.double() - RP.double()).norm() / RP.double().norm()) <= 1e-7


@pytest.mark.parametrize("rule", ["nm_adam_update", "nm_adamh_update"])
def test_row_blocks_against_the_reference_library(rule):
    """Row blocks (own learning-rate multipliers, a frozen block, per-block AdamH norms) through both libraries' one-tensor
    entry points: moments bit-equal, parameters bit-equal for Adam and within 1e-6 for AdamH."""
    if not os.path.exists(REF_OPT):
        pytest.skip("oracle/_ref/libref_optim.so was not built (make -C oracle _ref/libref_optim.so)")
    import ctypes
    from gpu_common import lib, nmce
    rdll = ctypes.CDLL(REF_OPT)
    getattr(rdll, rule).restype, getattr(rdll, rule).argtypes = nmce.SIGS[rule]
    rng = np.random.default_rng(11)
    R, C = 200, 72
    p = (rng.standard_normal((R, C)) * 0.02).astype(np.float32)
    g = (rng.standard_normal((R, C)) * 1e-3).astype(np.float32)
    mu = (rng.standard_normal((R, C)) * 1e-4).astype(np.float32)
    nu = ((rng.standard_normal((R, C)) * 1e-3) ** 2).astype(np.float32)
    bor = torch.from_numpy(rng.integers(0, 4, R).astype(np.int32)).cuda()
    mult = torch.tensor([0.5, 1.0, 2.0, 0.25], dtype=torch.float32, device="cuda")
    frozen = torch.tensor([0, 0, 1, 0], dtype=torch.uint8, device="cuda")
    out = []
    for fn in (lib().raw(rule), getattr(rdll, rule)):
        P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
        assert fn(nmce.ptr(P), None, nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), R, C, 1, 0.01, 0.9, 0.98, 1e-20, 0.0, 0, 1.0,
                  nmce.ptr(bor), nmce.ptr(mult), nmce.ptr(frozen), 4, None) == 0
        torch.cuda.synchronize()
        out.append((P, M, V))
    (P, M, V), (RP, RM, RV) = out
    assert torch.equal(M, RM) and torch.equal(V, RV)
    if rule == "nm_adam_update":
        assert torch.equal(P, RP)
    else:
        assert float((P.double() - RP.double()).norm() / RP.double().norm()) <= 1e-6

"""GPU parity tests of the fused linear cross-entropy, through the C ABI, against the CPU oracle (oracle/ce_ref.c,
float32) on identical seeded, bf16-rounded inputs. Bars (the parity contract): scalar loss relative error <= 1e-4,
per-token loss and lse within 2e-5 nats, dX and dW relative L2 error <= 3e-3 with cosine >= 0.9999, ignored rows
exactly zero. The case list follows the reference's tests/s5/test_ce.py (grad cases, odd shapes, bitwise invariants,
in-place and accumulating dX, strict dW, f32 store, f32 io, grad_scale, loss_partial tree) plus the extensions
(z-loss, ignore index, Zipf labels)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle():
    from gpu_common import O
    if not hasattr(_oracle, "c"):
        _oracle.c = O.COracle()
    return _oracle.c


def check_case(x, w, y, wt, *, z_loss=0.0, ignore_index=None, chunk=1024, impl="B1", store=1, bias=None, io_f32=False,
               tag=""):
    """Runs oracle and kernel on the same inputs and applies the parity bars. Returns the kernel outputs."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_REL, LOSS_TOK, cos, grad_scale_dev, rel, run_ce, to_dev
    dt = torch.float32 if io_f32 else torch.bfloat16
    X, W, Y, WT = to_dev(x, w, y, wt, dt)
    valid = (y >= 0) & (y < w.shape[0])
    if ignore_index is not None:
        valid &= y != ignore_index
    gs = grad_scale_dev(torch.from_numpy((wt * valid).astype(np.float32)).cuda())
    g = float(gs.item())
    # the oracle with float64 accumulators on the same float32 inputs: its float32-accumulating twin carries ~1e-5 of its
    # own summation noise in lse at V = 128256, which is the size of the per-token bar
    ol, olse, odx, odw = _oracle().run(x, w, y, wt, g, z_loss=z_loss, ignore_index=ignore_index, bias=bias,
                                       f64acc=True)
    B = None if bias is None else torch.from_numpy(bias).cuda()
    kw = dict(z_loss=z_loss if z_loss else None, ignore_index=ignore_index, bias=B, store=store)
    loss, lse, dx, dw, lp = run_ce(X, W, Y, WT, gs, impl=impl, chunk=chunk, **kw)
    counts = valid & (wt != 0)
    lk, lsek = loss.cpu().numpy(), lse.cpu().numpy()
    assert np.abs(lk - ol).max() <= LOSS_TOK, f"{tag}: per-token loss {np.abs(lk - ol).max():.3e}"
    assert np.abs(lsek - olse).max() <= LOSS_TOK, f"{tag}: lse {np.abs(lsek - olse).max():.3e}"
    assert (lk[~counts] == 0).all(), f"{tag}: loss of an ignored row is not 0"
    if counts.any():
        s_k = float((lk.astype(np.float64) * wt).sum() * g)
        s_o = float((ol.astype(np.float64) * wt).sum() * g)
        assert abs(s_k - s_o) <= LOSS_REL * abs(s_o), f"{tag}: scalar loss {s_k} vs {s_o}"
        rx, cx = rel(dx, odx), cos(dx, odx)
        rw, cw = rel(dw, odw), cos(dw, odw)
        assert rx <= GRAD_REL and cx >= GRAD_COS, f"{tag}: dX rel {rx:.3e} cos {cx:.6f}"
        assert rw <= GRAD_REL and cw >= GRAD_COS, f"{tag}: dW rel {rw:.3e} cos {cw:.6f}"
    gz = (~valid) | (wt == 0)
    assert (dx.float().cpu().numpy()[gz] == 0).all(), f"{tag}: dX of an ignored row is not 0"
    if counts.any():
        print(f"[parity] {tag}: loss {np.abs(lk - ol).max():.2e} lse {np.abs(lsek - olse).max():.2e} "
              f"dX rel {rx:.2e} cos {cx:.7f} dW rel {rw:.2e} cos {cw:.7f}")
    return loss, lse, dx, dw, lp, gs


# ------------------------------------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("case", ["a", "b", "c"])
@pytest.mark.parametrize("store", [1, 0])
def test_golden_vectors_of_the_reference_oracle(golden, case, store):
    """Inputs and float64 outputs made by the reference's own numpy oracle (tests/golden/make_golden.py). Case b has
    logits ~ N(0, 9) (the reference's make_case scale): there p = exp(z_s - lse) from the bf16-rounded stored logit
    (part of the math contract, as in the reference's B1) moves p by up to |z| 2^-9, so with the bf16 store its
    gradients are held to 1e-2 against float64 and to the 3e-3 bar with the f32 store."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, cos, rel, run_ce, to_dev
    x, w, y, wt = (golden[f"{case}_{k}"] for k in ("x", "w", "labels", "weight"))
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = torch.tensor([1.0 / float(golden[f"{case}_denom"])], dtype=torch.float32, device="cuda")
    loss, lse, dx, dw, _ = run_ce(X, W, Y, WT, gs, chunk=64, store=store)
    on = wt != 0
    dl = np.abs(loss.cpu().numpy() - golden[f"{case}_loss"])[on].max()
    rx, cx = rel(dx, golden[f"{case}_grad_x"]), cos(dx, golden[f"{case}_grad_x"])
    rw, cw = rel(dw, golden[f"{case}_grad_w"]), cos(dw, golden[f"{case}_grad_w"])
    print(f"[parity] golden {case} store {'bf16' if store else 'f32'}: loss {dl:.2e} dX rel {rx:.2e} cos {cx:.7f} "
          f"dW rel {rw:.2e} cos {cw:.7f}")
    assert dl <= LOSS_TOK
    assert (loss.cpu().numpy()[~on] == 0).all()
    bar = 1e-2 if (case == "b" and store == 1) else GRAD_REL
    assert rx <= bar and cx >= GRAD_COS
    assert rw <= bar and cw >= GRAD_COS


# ------------------------------------------------------------------------------------------------ parity vs the oracle
@pytest.mark.parametrize("T,D,V,labels,z_loss,chunk", [
    (2125, 512, 8256, "uniform", 0.0, 1024),
    (2125, 1024, 8256, "uniform", 1e-4, 1024),
    (1500, 2048, 4096, "zipf", 1e-4, 512),
    (1300, 768, 64256, "uniform", 0.0, 1024),
    (513, 512, 128256, "uniform", 1e-4, 512),      # 1-row tail chunk at the full vocabulary
])
def test_parity_benchmark_distributions(T, D, V, labels, z_loss, chunk):
    from gpu_common import O
    x, w, y, wt = O.make_inputs(T, D, V, seed=T + D + V, ignore_frac=0.02, labels=labels)
    check_case(x, w, y, wt, z_loss=z_loss, chunk=chunk, tag=f"T{T} D{D} V{V} {labels}")


@pytest.mark.parametrize("T,D,V,chunk", [(700, 520, 1000, 256), (1025, 136, 8257, 1024), (1, 64, 130, 128),
                                         (2100, 512, 1000, 1022), (40, 8, 9, 16)])
def test_odd_shapes(T, D, V, chunk):
    """V not a multiple of 8 or 256, D not a multiple of 64, T below one chunk, a 1-row tail, 1022-row chunks
    (reference test_ce.py:337-367)."""
    from gpu_common import O
    x, w, y, wt = O.make_inputs(T, D, V, seed=V + T, ignore_frac=0.2 if T > 1 else 0.0, w_std=0.9 / D ** 0.5)
    check_case(x, w, y, wt, chunk=chunk, tag=f"odd T{T} D{D} V{V}")
    check_case(x, w, y, wt, chunk=chunk, store=0, z_loss=1e-3, tag=f"odd T{T} D{D} V{V} f32 store")


def test_wide_logits():
    """logits ~ N(0, 9) as the reference's make_case (tests/s5/nmce.py:111-122): the online-softmax rescaling and the
    bf16 logits store are exercised at a scale where they matter. The gradient bars are the oracle's with the bf16 store
    emulated (p from the rounded logit is part of the contract, include/marincpp/kernels/cross_entropy.hpp)."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, cos, grad_scale_dev, rel, run_ce, to_dev
    T, D, V = 1200, 512, 8256
    rng = np.random.default_rng(9)
    from gpu_common import O
    x = O.bf16_round(rng.standard_normal((T, D), dtype=np.float32))
    w = O.bf16_round(rng.standard_normal((V, D), dtype=np.float32) * np.float32(3.0 / D ** 0.5))
    y = rng.integers(0, V, size=T).astype(np.int32)
    wt = np.ones(T, np.float32)
    wt[::7] = 0
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    ol, olse, odx, odw = _oracle().run(x, w, y, wt, float(gs.item()), bf16_store=True, f64acc=True)
    loss, lse, dx, dw, _ = run_ce(X, W, Y, WT, gs)
    print(f"[parity] wide logits: loss {np.abs(loss.cpu().numpy() - ol).max():.2e} lse "
          f"{np.abs(lse.cpu().numpy() - olse).max():.2e} dX rel {rel(dx, odx):.2e} dW rel {rel(dw, odw):.2e}")
    assert np.abs(loss.cpu().numpy() - ol).max() <= 2 * LOSS_TOK     # |z| up to ~15: f32 accumulation order shows
    assert np.abs(lse.cpu().numpy() - olse).max() <= 2 * LOSS_TOK
    assert rel(dx, odx) <= GRAD_REL and cos(dx, odx) >= GRAD_COS
    assert rel(dw, odw) <= GRAD_REL and cos(dw, odw) >= GRAD_COS


def test_extensions_z_loss_and_ignore_index():
    from gpu_common import O
    x, w, y, wt = O.make_inputs(900, 512, 4000, seed=3, ignore_frac=0.1)
    y[5], wt[5] = 77, 1.0
    y[6], wt[6] = 4000, 1.0        # outside [0, V): ignored without any index
    check_case(x, w, y, wt, z_loss=1e-2, ignore_index=77, tag="z-loss + ignore index 77")
    check_case(x, w, y, wt, z_loss=0.0, ignore_index=-100, tag="ignore index -100")


# ------------------------------------------------------------------------------------------------ bitwise invariants
def test_bitwise_invariants():
    """Repeat runs give the same bits; loss, lse and dX do not depend on the chunk size; every implementation value
    runs the same pipeline; a forward-only call gives the loss of the gradient call (reference test_ce.py:173-208)."""
    from gpu_common import O, grad_scale_dev, rel, run_ce, same_bits, to_dev
    x, w, y, wt = O.make_inputs(3000, 512, 8256, seed=5, ignore_frac=0.1)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    a = run_ce(X, W, Y, WT, gs, chunk=1024)
    b = run_ce(X, W, Y, WT, gs, chunk=1024)
    for i, n in enumerate(("loss", "lse", "dx", "dw", "loss_partial")):
        assert same_bits(a[i], b[i]), f"repeat {n}"
    for ch in (128, 512, 4096):
        c = run_ce(X, W, Y, WT, gs, chunk=ch)
        for i, n in enumerate(("loss", "lse", "dx")):
            assert same_bits(c[i], a[i]), f"chunk {ch} vs 1024 {n}"
        assert rel(c[3], a[3]) < 1e-5, f"chunk {ch}: dW may differ only by summation order"
    for impl in ("A", "B1.5", "B2"):
        c = run_ce(X, W, Y, WT, gs, chunk=1024, impl=impl)
        for i, n in enumerate(("loss", "lse", "dx", "dw", "loss_partial")):
            assert same_bits(c[i], a[i]), f"{impl} vs B1 {n}"
    f = run_ce(X, W, Y, WT, gs, chunk=1024, fwd=True)
    assert same_bits(f[0], a[0]) and same_bits(f[1], a[1]) and same_bits(f[4], a[4])
    # lse == NULL is allowed (the workspace lse is used); dx == NULL / dw == NULL select one gradient
    from gpu_common import lib, nmce
    loss2 = torch.empty_like(a[0])
    dw2 = torch.zeros_like(a[3])
    ws = nmce.Ws.get(lib().nm_ce_workspace_bytes(1, 3000, 512, 8256, 1024, 1))
    lib().nm_fused_linear_ce(1, 0, 1, 1, nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(gs), None,
                             nmce.ptr(loss2), None, None, None, 0, nmce.ptr(dw2), None, 0, 0, 3000, 512, 8256, 1024,
                             nmce.ptr(ws), None)
    torch.cuda.synchronize()
    assert same_bits(loss2, a[0]) and same_bits(dw2, a[3])


def test_inplace_and_accumulating_dx():
    from gpu_common import O, grad_scale_dev, nmce, rel, run_ce, same_bits, to_dev
    x, w, y, wt = O.make_inputs(2500, 768, 8256, seed=6, ignore_frac=0.1)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    a = run_ce(X, W, Y, WT, gs)
    xi = X.clone()
    r = run_ce(xi, W, Y, WT, gs, dx=xi)
    assert same_bits(xi, a[2]) and same_bits(r[3], a[3]), "dx == x must equal a separate dX"
    g = torch.Generator(device="cuda").manual_seed(70)
    old = (torch.randn(2500, 768, generator=g, device="cuda") * 3e-4).to(torch.bfloat16)
    lev = old.clone()
    run_ce(X, W, Y, WT, gs, dx=lev, acc_dx=True, rounding=nmce.LEV)
    assert same_bits(lev, (old.float() + a[2].float()).to(torch.bfloat16)), "levanter: bf16(old + f32(bf16(acc)))"
    acc = old.clone()
    run_ce(X, W, Y, WT, gs, dx=acc, acc_dx=True, rounding=nmce.ACC)
    from gpu_common import grad_scale_dev as _  # noqa: F401
    odx = _oracle().run(x, w, y, wt, float(gs.item()), want_dw=False)[2]
    want = torch.from_numpy(odx).cuda().double() + old.double()
    assert rel(acc, want) < rel(lev, want), "accurate accumulate must be closer to the truth than the levanter form"
    assert (acc.view(torch.int16) != lev.view(torch.int16)).double().mean().item() > 1e-3
    with pytest.raises(nmce.NmError):   # dx == x cannot accumulate (reference ce_api.cpp:142)
        run_ce(xi, W, Y, WT, gs, dx=xi, acc_dx=True)


def test_strict_dw_and_finish_microbatch():
    """dw_round = 1: each chunk's dW is rounded to bf16 into the microbatch accumulator; finish adds its bf16 rounding
    into dw and clears it (reference test_ce.py:275-302)."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, same_bits, to_dev
    V, D, chunk = 8256, 512, 1024
    dw = (torch.randn(V, D, device="cuda") * 1e-3).float()
    want = dw.clone()
    mb = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    for micro in range(2):
        T = 2 * chunk + 300
        x, w, y, wt = O.make_inputs(T, D, V, seed=80 + micro, ignore_frac=0.1)
        X, W, Y, WT = to_dev(x, w, y, wt)
        gs = grad_scale_dev(WT)
        run_ce(X, W, Y, WT, gs, chunk=chunk, dw=dw, dw_mb=mb, dw_round=1)
        lib().nm_ce_finish_microbatch(nmce.ptr(dw), nmce.ptr(mb), V * D, None)
        acc = torch.zeros(V, D, dtype=torch.float32, device="cuda")
        for r0 in range(0, T, chunk):
            r1 = min(T, r0 + chunk)
            dwc = run_ce(X[r0:r1].contiguous(), W, Y[r0:r1].contiguous(), WT[r0:r1].contiguous(), gs, chunk=chunk)[3]
            acc += dwc.to(torch.bfloat16).float()
        want = want + acc.to(torch.bfloat16).float()
    torch.cuda.synchronize()
    assert same_bits(dw, want)
    assert bool((mb == 0).all())


def test_f32_io_config0():
    """BASELINE config 0 in full: 512 tokens, f32 x (RMS-normalised N(0,1)) and f32 W ~ N(0, 0.02) at D 512,
    V 128256, labels uniform with 5% set to -100, z-loss 0, mean over non-ignored tokens; implementation A, io f32."""
    from gpu_common import O
    x, w, y, wt = O.make_inputs(512, 512, 128256, seed=0xC0, ignore_frac=0.05, bf16=False)
    check_case(x, w, y, wt, impl="A", io_f32=True, chunk=512, tag="config 0")


def test_f32_io_with_bias():
    from gpu_common import O
    x, w, y, wt = O.make_inputs(700, 256, 2000, seed=9, ignore_frac=0.1, bf16=False, w_std=0.06)
    bias = np.random.default_rng(90).standard_normal(2000).astype(np.float32)
    check_case(x, w, y, wt, impl="A", io_f32=True, chunk=256, bias=bias, store=0, tag="f32 io + bias")
    xb, wb = O.bf16_round(x), O.bf16_round(w)
    check_case(xb, wb, y, wt, impl="A", chunk=256, bias=bias, tag="bf16 io + bias")


def test_grad_scale_and_loss_partial_bits(golden):
    """mult / sum(w) exact values (reference test_ce.py:587-599) and the per-chunk loss tree against its emulation."""
    from gpu_common import O, grad_scale_dev, lib, nmce
    for B in (128, 256):
        wt = torch.ones(B, 4096, dtype=torch.float32, device="cuda")
        wt[:, -1] = 0
        assert grad_scale_dev(wt).item() == float(golden[f"grad_scale_B{B}"])
    g = torch.Generator(device="cuda").manual_seed(3)
    wt = (torch.rand(524288, generator=g, device="cuda") < 0.9).float()
    assert grad_scale_dev(wt).item() == float(np.float32(1.0) / np.float32(wt.sum().item()))
    tl, tw = golden["tree_loss"], golden["tree_weight"]
    x, w, y, wgt = O.make_inputs(5000, 64, 500, seed=1, ignore_frac=0.07)
    from gpu_common import run_ce, to_dev
    X, W, Y, WT = to_dev(x, w, y, wgt)
    gs = grad_scale_dev(WT)
    for chunk in (1024, 2048, 4096):
        loss, _, _, _, lp = run_ce(X, W, Y, WT, gs, chunk=chunk)
        want = O.chunk_loss_tree(loss.cpu().numpy(), wgt, chunk)
        assert lp.cpu().numpy().tobytes() == want.tobytes(), f"loss_partial bits, chunk {chunk}"


def test_workspace_guard_band_and_status():
    """A workspace of exactly nm_ce_workspace_bytes followed by a guard band that must stay untouched (reference
    test_ce.py:312-321), for the bf16 and f32 stores and for implementation A's f32-io layout."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, to_dev
    T, D, V, chunk = 1700, 512, 8256, 512
    x, w, y, wt = O.make_inputs(T, D, V, seed=9)
    for impl, store, f32 in (("B1", 1, False), ("B1", 0, False), ("A", 0, True)):
        X, W, Y, WT = to_dev(x, w, y, wt, torch.float32 if f32 else torch.bfloat16)
        gs = grad_scale_dev(WT)
        nb = lib().nm_ce_workspace_bytes(nmce.IMPLS[impl], T, D, V, chunk, store)
        guard = 1 << 20
        wsb = torch.full((nb + guard,), 0xA5, dtype=torch.uint8, device="cuda")
        run_ce(X, W, Y, WT, gs, impl=impl, chunk=chunk, store=store, ws=wsb[:nb])
        assert bool((wsb[nb:] == 0xA5).all()), f"{impl} store {store}: the call wrote past nm_ce_workspace_bytes"
        status = ctypes.c_uint32(7)
        lib().nm_ce_device_status(nmce.ptr(wsb), None, ctypes.byref(status))
        assert status.value == 0


def test_argument_errors_on_device():
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, to_dev
    x, w, y, wt = O.make_inputs(64, 64, 300, seed=2)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    B = torch.zeros(300, device="cuda")
    with pytest.raises(nmce.NmError) as e:      # logit_bias only with implementation A
        run_ce(X, W, Y, WT, gs, impl="B1", bias=B)
    assert e.value.status == 1
    with pytest.raises(nmce.NmError) as e:      # gradients need grad_scale
        run_ce(X, W, Y, WT, None)
    assert e.value.status == 1
    with pytest.raises(nmce.NmError) as e:      # strict dW needs dw_microbatch
        run_ce(X, W, Y, WT, gs, dw_round=1)
    assert e.value.status == 1
    assert lib().nm_ce_device_arch() == 100 and lib().nm_device_arch() == 100
    # pointers the kernels access with 16-byte vectors or TMA must be 16-byte aligned: refused on the host, no launch
    big = torch.zeros(64 * 64 + 8, dtype=torch.bfloat16, device="cuda")
    odd_dx = big[4:4 + 64 * 64].view(64, 64)               # 8 bytes past a 16-byte boundary
    with pytest.raises(nmce.NmError) as e:
        run_ce(X, W, Y, WT, gs, dx=odd_dx)
    assert e.value.status == 1 and "16-byte aligned" in str(e.value)
    odd_x = big[4:4 + 64 * 64].view(64, 64)
    with pytest.raises(nmce.NmError) as e:
        run_ce(odd_x, W, Y, WT, gs)
    assert e.value.status == 1 and "16-byte aligned" in str(e.value)
    from gpu_common import lib as _lib
    with pytest.raises(nmce.NmError) as e:                  # the RMSNorm entry point checks its row pointers too
        _lib().nm_rmsnorm_fwd(1, 0, nmce.ptr(odd_x), nmce.ptr(big), nmce.ptr(big), nmce.ptr(torch.zeros(64, device="cuda")),
                              64, 64, 1e-5, None)
    assert e.value.status == 1 and "16-byte aligned" in str(e.value)


def test_bounded_wait_times_out_and_reports():
    """The failure path of the device-side waits, made on purpose in the one safe way: a wait on a barrier that nothing
    completes, limited to a million clocks. It must end by itself, set its status bit, wake the other waiter through
    the abort flag, and leave the context usable (the next CE call works and reports a clean status)."""
    from gpu_common import O, grad_scale_dev, lib, nmce, run_ce, to_dev
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    saw = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib().nm_ce_test_wait_timeout(nmce.ptr(status), 1_000_000, nmce.ptr(saw), None)
    torch.cuda.synchronize()
    assert int(status.item()) == 4, f"expected the epilogue-wait bit, got {int(status.item())}"
    assert int(saw.item()) == 1, "the second waiter did not leave through the abort flag"
    with pytest.raises(nmce.NmError):            # limits beyond a millisecond are refused
        lib().nm_ce_test_wait_timeout(nmce.ptr(status), 10**9, nmce.ptr(saw), None)
    # a status word with a bit set is what nm_ce_device_status turns into NM_ERR_DEVICE
    fake_ws = torch.zeros(64, dtype=torch.int32, device="cuda")
    fake_ws[0] = 4
    st = ctypes.c_uint32(0)
    with pytest.raises(nmce.NmError) as e:
        lib().nm_ce_device_status(nmce.ptr(fake_ws), None, ctypes.byref(st))
    assert e.value.status == 2 and st.value == 4
    x, w, y, wt = O.make_inputs(300, 64, 500, seed=8)
    X, W, Y, WT = to_dev(x, w, y, wt)
    run_ce(X, W, Y, WT, grad_scale_dev(WT), chunk=128)      # the context is still healthy


def test_dlogits_entry_point():
    """nm_ce_dlogits alone over a bf16 store: n = g (exp(z_s - lse) - onehot), columns >= V zeroed."""
    from gpu_common import lib, nmce, rel
    rows, V = 300, 1003
    ldS = (V + 7) // 8 * 8
    g = torch.Generator(device="cuda").manual_seed(4)
    z = torch.randn(rows, ldS, generator=g, device="cuda").to(torch.bfloat16)
    lse = torch.logsumexp(z[:, :V].float(), dim=1)
    gsc = torch.rand(rows, generator=g, device="cuda") + 0.5
    tg = torch.randint(0, V, (rows,), generator=g, device="cuda", dtype=torch.int32)
    want = torch.exp(z[:, :V].float() - lse[:, None]) * gsc[:, None]
    want[torch.arange(rows), tg.long()] -= gsc
    store = z.clone()
    lib().nm_ce_dlogits(1, nmce.ptr(store), ldS, nmce.ptr(lse), nmce.ptr(gsc), nmce.ptr(tg), rows, V, None)
    torch.cuda.synchronize()
    assert rel(store[:, :V], want) < 3e-3
    assert bool((store[:, V:] == 0).all())


# ------------------------------------------------------------------------------------------------ full-size properties
@pytest.mark.parametrize("T,D,labels,chunk", [(131072, 512, "uniform", 16384), (65536, 2048, "zipf", 16384)])
def test_full_size_properties(T, D, labels, chunk):
    """BASELINE shapes at V = 128256 through size-independent properties: (1) a row subsample against the oracle (rows
    are independent); (2) the softmax gradient sums to zero over the vocabulary, so the column sums of dW equal
    sum_t g_t 2 L lse_t x_t; (3) dW is additive over row ranges; (4) ignored rows are exactly zero; (5) loss_partial
    sums to the weighted loss."""
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, cos, grad_scale_dev, rel, run_ce
    V, L = 128256, 1e-4
    g = torch.Generator(device="cuda").manual_seed(0xC1 + D)
    X = torch.randn(T, D, generator=g, device="cuda")
    X = (X / X.pow(2).mean(dim=1, keepdim=True).sqrt()).to(torch.bfloat16)
    W = (torch.randn(V, D, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    if labels == "uniform":
        Y = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    else:
        from gpu_common import O
        u = torch.rand(T, generator=g, device="cuda").cpu().numpy()
        Y = torch.from_numpy(O.zipf_labels(u, V, 1.1).astype(np.int32)).cuda()
    Y[torch.rand(T, generator=g, device="cuda") < 0.02] = -100
    WT = (Y != -100).float()
    gs = grad_scale_dev(WT)
    loss, lse, dx, dw, lp = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=L)
    # (1) subsample
    n = 192
    ol, olse, odx, _ = _oracle().run(X[:n].float().cpu().numpy(), W.float().cpu().numpy(), Y[:n].cpu().numpy(),
                                     WT[:n].cpu().numpy(), float(gs.item()), z_loss=L, want_dw=False, f64acc=True)
    assert np.abs(loss[:n].cpu().numpy() - ol).max() <= LOSS_TOK
    assert np.abs(lse[:n].cpu().numpy() - olse).max() <= LOSS_TOK
    assert rel(dx[:n], odx) <= GRAD_REL and cos(dx[:n], odx) >= GRAD_COS
    # (2) column sums of dW
    gt = WT * gs
    want_cols = ((gt * 2 * L * lse)[:, None].double() * X.double()).sum(dim=0)
    got_cols = dw.double().sum(dim=0)
    scale = dw.double().abs().sum(dim=0)     # the sums cancel: compare against the magnitude that was summed
    assert float(((got_cols - want_cols).abs() / scale).max()) < 2e-3
    # (3) additivity over row ranges (same grad_scale)
    h = T // 2
    d1 = run_ce(X[:h], W, Y[:h], WT[:h], gs, chunk=chunk, z_loss=L)[3]
    d2 = run_ce(X[h:], W, Y[h:], WT[h:], gs, chunk=chunk, z_loss=L)[3]
    assert rel(d1 + d2, dw) < 1e-5
    del d1, d2
    # (4), (5)
    ign = WT == 0
    assert bool((loss[ign] == 0).all()) and bool((dx[ign].float() == 0).all())
    assert abs(float(lp.double().sum()) - float((loss.double() * WT).sum())) <= 1e-6 * float(lp.double().sum())
    assert torch.isfinite(dw).all() and torch.isfinite(dx.float()).all()


def test_cuda_graph_capture_and_replay():
    """The call allocates nothing and never synchronises, so it can be captured into a CUDA graph (as the reference
    trainer captures its whole step, src/train/trainer.cpp:155-163); replays give the bits of the eager call."""
    from gpu_common import O, grad_scale_dev, lib, nmce, same_bits, to_dev
    T, D, V, chunk = 2500, 512, 8256, 1024
    x, w, y, wt = O.make_inputs(T, D, V, seed=31, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    ws = torch.empty(lib().nm_ce_workspace_bytes(1, T, D, V, chunk, 1), dtype=torch.uint8, device="cuda")
    outs = {}
    for name in ("eager", "graph"):
        outs[name] = dict(loss=torch.zeros(T, device="cuda"), lse=torch.zeros(T, device="cuda"),
                          dx=torch.zeros_like(X), dw=torch.zeros(V, D, device="cuda"),
                          lp=torch.zeros((T + chunk - 1) // chunk, device="cuda"))

    def call(o, stream):
        lib().nm_fused_linear_ce_ex(1, 0, 1, 1, nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(gs), None,
                                    nmce.ptr(o["loss"]), nmce.ptr(o["lse"]), nmce.ptr(o["lp"]), nmce.ptr(o["dx"]), 0,
                                    nmce.ptr(o["dw"]), None, 0, 0, T, D, V, chunk, nmce.ptr(ws),
                                    ctypes.c_void_p(stream), 1e-4, -100, None)

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        call(outs["eager"], s.cuda_stream)      # eager first: one-time set-up happens outside any capture
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        call(outs["graph"], s.cuda_stream)
    for _ in range(3):                          # dW accumulates: compare after the same number of adds
        outs["graph"]["dw"].zero_()
        g.replay()
    torch.cuda.synchronize()
    for k in ("loss", "lse", "dx", "dw", "lp"):
        assert same_bits(outs["graph"][k], outs["eager"][k]), f"graph replay differs from the eager call: {k}"


def test_two_devices_same_bits():
    """The same call on GPU 0 and GPU 1 of one process gives the same bits (reference test_ce.py:553-574)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from gpu_common import O, grad_scale_dev, run_ce, same_bits, to_dev
    x, w, y, wt = O.make_inputs(1500, 512, 8256, seed=12)
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            X, W, Y, WT = (t.to(f"cuda:{dev}") for t in to_dev(x, w, y, wt))
            gs = torch.empty(1, dtype=torch.float32, device=f"cuda:{dev}")
            from gpu_common import lib, nmce
            lib().nm_ce_grad_scale(nmce.ptr(WT), WT.numel(), 1.0, nmce.ptr(gs), None)
            dx = torch.empty_like(X)
            dw = torch.zeros(8256, 512, dtype=torch.float32, device=f"cuda:{dev}")
            loss, lse = nmce.ce_call(lib(), "B1", X, W, Y, WT, gs, dx=dx, dw=dw)
            torch.cuda.synchronize()
            outs.append([t.cpu() for t in (loss, lse, dx, dw)])
    for a, b in zip(*outs):
        assert same_bits(a, b)


def test_suggested_chunk_rows():
    """nm_ce_suggest_chunk_rows: min(T, 128 x SM count), so that the tiles of a full chunk fill whole waves."""
    from gpu_common import lib
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert lib().nm_ce_suggest_chunk_rows(131072) == min(131072, 128 * sms)
    assert lib().nm_ce_suggest_chunk_rows(1000) == 1000
    assert lib().nm_ce_suggest_chunk_rows(0) == 1


@pytest.mark.parametrize("T,D,V,chunk", [(3000, 512, 8256, 1024), (2500, 1024, 16400, 2500), (700, 2048, 8256, 512)])
def test_cta_pairs_give_the_same_bits(T, D, V, chunk):
    """One CTA per tile and a CTA pair per tile (tcgen05 cta_group::2) add the same products in the same order: every
    output is bit-identical, for each of the three contractions separately and for all together, on ragged shapes."""
    from gpu_common import O, grad_scale_dev, lib, run_ce, same_bits, to_dev
    x, w, y, wt = O.make_inputs(T, D, V, seed=17, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    try:
        lib().nm_ce_set_cta_pair(0, 0, 0)
        a = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4)
        for mode in ((1, 0, 0), (0, 1, 0), (0, 0, 1), (1, 1, 1)):
            lib().nm_ce_set_cta_pair(*mode)
            b = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4)
            for i, n in enumerate(("loss", "lse", "dx", "dw", "loss_partial")):
                assert same_bits(a[i], b[i]), f"pairs {mode}: {n} differs"
    finally:
        lib().nm_ce_set_cta_pair(-1, -1, -1)     # back to the per-launch choice


@pytest.mark.parametrize("T,D,V,chunk", [(1000, 264, 1001, 384), (130, 512, 8256, 64), (2049, 1024, 640, 2049)])
def test_outputs_stay_inside_their_buffers(T, D, V, chunk):
    """Every output (dx, dw, loss, lse, loss_partial) sits between two guard bands of 0xA5 bytes that must survive the
    call, on ragged shapes (rows, columns and the vocabulary not multiples of the tile sizes): the TMA stores and
    reductions clip at the tensor extents, the direct stores are predicated."""
    from gpu_common import O, grad_scale_dev, lib, nmce, to_dev
    x, w, y, wt = O.make_inputs(T, D, V, seed=23, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    G = 4096
    n_chunks = (T + chunk - 1) // chunk

    def guarded(nbytes):
        buf = torch.full((G + nbytes + G,), 0xA5, dtype=torch.uint8, device="cuda")
        return buf, buf[G:G + nbytes]

    bufs = {"dx": guarded(T * D * 2), "dw": guarded(V * D * 4), "loss": guarded(T * 4), "lse": guarded(T * 4),
            "lp": guarded(n_chunks * 4)}
    bufs["dw"][1].zero_()
    ws = nmce.Ws.get(lib().nm_ce_workspace_bytes(1, T, D, V, chunk, 1))
    p = {k: ctypes.c_void_p(v[1].data_ptr()) for k, v in bufs.items()}
    lib().nm_fused_linear_ce(1, 0, 1, 1, nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(gs), None,
                             p["loss"], p["lse"], p["lp"], p["dx"], 0, p["dw"], None, 0, 0, T, D, V, chunk,
                             nmce.ptr(ws), None)
    torch.cuda.synchronize()
    for name, (buf, view) in bufs.items():
        n = view.numel()
        assert bool((buf[:G] == 0xA5).all()) and bool((buf[G + n:] == 0xA5).all()), f"{name}: a guard band was written"
    dw = bufs["dw"][1].view(torch.float32).view(V, D)
    dx = bufs["dx"][1].view(torch.bfloat16).view(T, D)
    assert bool(torch.isfinite(dw).all()) and bool(torch.isfinite(dx.float()).all())
    assert float(dw.abs().sum()) > 0 and float(dx.float().abs().sum()) > 0

"""The readout head entry point (RMSNorm -> fused CE with dX written over the norm output -> RMSNorm backward added
into d_state, gain partials) against the composed C-ABI calls, bit for bit, as the reference's readout case does
(tests/s5/test_ce.py:379-460): full and partial visible width, gain-only, no backbone gradient, forward-only, both
roundings; the RMSNorm pair alone against a float64 torch reference; one float64 autograd check of the whole head."""
import pytest
import torch

pytestmark = pytest.mark.gpu
EPS = 1e-5


def _inputs(T, D, V, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    state = (torch.randn(T, D, generator=g, device="cuda") * 2).to(torch.bfloat16)
    gain = (1.0 + 0.2 * torch.randn(D, generator=g, device="cuda")).to(torch.bfloat16)
    W = (torch.randn(V, D, generator=g, device="cuda") * (0.9 / D ** 0.5)).to(torch.bfloat16)
    tg = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    w = torch.ones(T, dtype=torch.float32, device="cuda")
    w[::7] = 0
    w[-1] = 0
    gs = torch.tensor([0.37 / float(w.sum().item())], dtype=torch.float32, device="cuda")
    return g, state, gain, W, tg, w, gs


@pytest.mark.parametrize("D", [512, 1024, 136])
@pytest.mark.parametrize("rounding", [0, 1])
def test_rmsnorm_pair_against_float64(D, rounding):
    from gpu_common import lib, nmce, rel
    T = 777
    g, state, gain, *_ = _inputs(T, D, 64, seed=D)
    y = torch.empty_like(state)
    rstd = torch.empty(T, dtype=torch.float32, device="cuda")
    lib().nm_rmsnorm_fwd(1, rounding, nmce.ptr(state), nmce.ptr(gain), nmce.ptr(y), nmce.ptr(rstd), T, D, EPS, None)
    st = state.double().requires_grad_(True)
    gn = gain.double().requires_grad_(True)
    r64 = torch.rsqrt((st * st).mean(dim=1, keepdim=True) + EPS)
    y64 = st * r64 * gn
    dy = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(torch.bfloat16)
    dres = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(torch.bfloat16)
    (y64 * dy.double()).sum().backward()
    torch.cuda.synchronize()
    assert rel(rstd, r64[:, 0]) < 1e-6
    assert rel(y, y64) < 4e-3                       # bf16 output (two roundings under levanter)
    P = lib().nm_norm_partial_rows(T)
    assert 1 <= P <= 1024
    part = torch.zeros(P, D, dtype=torch.float32, device="cuda")
    dx = torch.empty_like(state)
    lib().nm_rmsnorm_bwd_add_partial(1, rounding, nmce.ptr(dy), nmce.ptr(state), nmce.ptr(gain), nmce.ptr(rstd),
                                     nmce.ptr(dres), nmce.ptr(dx), nmce.ptr(part), T, D, EPS, None)
    torch.cuda.synchronize()
    assert rel(dx, st.grad + dres.double()) < 6e-3  # bf16(dres + bf16(dx)) under levanter
    assert rel(part.sum(0), gn.grad) < 6e-3
    # in place over the residual gradient, and without a residual
    dres2 = dres.clone()
    lib().nm_rmsnorm_bwd_add_partial(1, rounding, nmce.ptr(dy), nmce.ptr(state), nmce.ptr(gain), nmce.ptr(rstd),
                                     nmce.ptr(dres2), nmce.ptr(dres2), None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert torch.equal(dres2, dx)
    dx0 = torch.empty_like(state)
    lib().nm_rmsnorm_bwd_add_partial(1, rounding, nmce.ptr(dy), nmce.ptr(state), nmce.ptr(gain), None, None,
                                     nmce.ptr(dx0), None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert rel(dx0, st.grad) < 6e-3


def test_readout_equals_composed_calls():
    from gpu_common import lib, nmce, same_bits
    V, D, T, chunk = 8256, 512, 2100, 1024
    g, state, gain, W, tg, w, gs = _inputs(T, D, V, seed=12)
    L = lib()
    P = L.nm_norm_partial_rows(T)
    for rounding in (nmce.LEV, nmce.ACC):
        for vis, with_state, with_gain, fwd_only in ((D, 1, 1, 0), (D // 2 + 64, 1, 1, 0), (D, 0, 1, 0), (D, 1, 0, 0),
                                                     (D, 0, 0, 0), (D, 1, 1, 1)):
            tag = f"rounding {rounding} vis {vis} d_state {with_state} gain {with_gain} fwd {fwd_only}"
            # composed reference
            y = torch.empty_like(state)
            rstd = torch.empty(T, dtype=torch.float32, device="cuda")
            L.nm_rmsnorm_fwd(1, rounding, nmce.ptr(state), nmce.ptr(gain), nmce.ptr(y), nmce.ptr(rstd), T, D, EPS, None)
            if vis < D:
                y[:, vis:] = 0
            dyr = torch.empty_like(y)
            dwr = torch.zeros(V, D, dtype=torch.float32, device="cuda")
            lr, lser = nmce.ce_call(L, "B1", y, W, tg, w, gs, chunk=chunk, dx=None if fwd_only else dyr,
                                    dw=None if fwd_only else dwr, forward_only=bool(fwd_only), rounding=rounding)
            d0 = (torch.randn(T, D, generator=g, device="cuda") * 1e-3).to(torch.bfloat16)
            dsr = d0.clone()
            pr = torch.zeros(P, D, dtype=torch.float32, device="cuda")
            if not fwd_only:
                if vis < D:
                    dyr[:, vis:] = 0
                scratch = torch.empty_like(state)
                L.nm_rmsnorm_bwd_add_partial(1, rounding, nmce.ptr(dyr), nmce.ptr(state), nmce.ptr(gain),
                                             nmce.ptr(rstd), nmce.ptr(dsr) if with_state else None,
                                             nmce.ptr(dsr if with_state else scratch), nmce.ptr(pr), T, D, EPS, None)
            # the entry point
            nout = torch.empty_like(state)
            nr = torch.empty(T, dtype=torch.float32, device="cuda")
            dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
            ds = d0.clone()
            pp = torch.zeros(P, D, dtype=torch.float32, device="cuda")
            loss = torch.empty(T, dtype=torch.float32, device="cuda")
            lse = torch.empty(T, dtype=torch.float32, device="cuda")
            ws = nmce.Ws.get(L.nm_ce_workspace_bytes(1, T, D, V, chunk, 1))
            L.nm_ce_readout(1, rounding, 1, nmce.ptr(state), nmce.ptr(gain), nmce.ptr(nr), nmce.ptr(nout), nmce.ptr(W),
                            nmce.ptr(dw), nmce.ptr(pp) if with_gain else None, nmce.ptr(gs),
                            nmce.ptr(ds) if with_state else None, vis, nmce.ptr(tg), nmce.ptr(w), nmce.ptr(loss),
                            nmce.ptr(lse), None, fwd_only, T, D, V, chunk, EPS, nmce.ptr(ws), None)
            torch.cuda.synchronize()
            assert same_bits(loss, lr) and same_bits(lse, lser), tag
            if not fwd_only:
                assert same_bits(dw, dwr), f"{tag}: dW"
                if with_state:
                    assert same_bits(ds, dsr), f"{tag}: d_state"
                else:
                    assert same_bits(ds, d0), f"{tag}: d_state must stay untouched"
                if with_gain:
                    assert same_bits(pp, pr), f"{tag}: gain partials"
                if not with_state and not with_gain:
                    assert same_bits(nout, y), f"{tag}: the norm output must be kept when no dY is needed"


def test_readout_against_float64_autograd():
    from gpu_common import lib, nmce, rel
    V, D, T, chunk = 8256, 512, 2100, 1024
    g, state, gain, W, tg, w, gs = _inputs(T, D, V, seed=12)
    L = lib()
    P = L.nm_norm_partial_rows(T)
    st = state.double().requires_grad_(True)
    gn = gain.double().requires_grad_(True)
    W64 = W.double().requires_grad_(True)
    yy = st * torch.rsqrt((st * st).mean(dim=1, keepdim=True) + EPS) * gn
    ce = torch.nn.functional.cross_entropy(yy @ W64.T, tg.long(), reduction="none")
    (ce * w.double() * gs.item()).sum().backward()
    nout = torch.empty_like(state)
    nr = torch.empty(T, dtype=torch.float32, device="cuda")
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")
    ds = torch.zeros_like(state)
    pp = torch.zeros(P, D, dtype=torch.float32, device="cuda")
    loss = torch.empty(T, dtype=torch.float32, device="cuda")
    ws = nmce.Ws.get(L.nm_ce_workspace_bytes(1, T, D, V, chunk, 1))
    L.nm_ce_readout(1, nmce.LEV, 1, nmce.ptr(state), nmce.ptr(gain), nmce.ptr(nr), nmce.ptr(nout), nmce.ptr(W),
                    nmce.ptr(dw), nmce.ptr(pp), nmce.ptr(gs), nmce.ptr(ds), D, nmce.ptr(tg), nmce.ptr(w),
                    nmce.ptr(loss), None, None, 0, T, D, V, chunk, EPS, nmce.ptr(ws), None)
    torch.cuda.synchronize()
    r_s, r_g, r_w = rel(ds, st.grad), rel(pp.sum(0), gn.grad), rel(dw, W64.grad)
    print(f"[parity] readout vs f64 autograd: d_state rel {r_s:.2e} dgain rel {r_g:.2e} dW rel {r_w:.2e}")
    assert r_s < 2e-2 and r_g < 2e-2 and r_w < 2e-2     # the reference's bars for this check (test_ce.py:459)


def test_readout_in_a_cuda_graph():
    """The whole readout (RMSNorm forward on the batch ring, fused CE, RMSNorm backward with gain partials) captured into
    a CUDA graph after one eager call on the device (the norm kernels look up their status word on first use) and
    replayed: the replay must give the eager call's bits, and the norm status word must stay clear."""
    import ctypes
    from gpu_common import lib, nmce, same_bits
    V, D, T, chunk = 8256, 512, 2100, 1024
    g, state, gain, W, tg, w, gs = _inputs(T, D, V, seed=21)
    L = lib()
    P = L.nm_norm_partial_rows(T)
    ws = torch.empty(L.nm_ce_workspace_bytes(1, T, D, V, chunk, 1) + 256, dtype=torch.uint8, device="cuda")
    d0 = (torch.randn(T, D, generator=g, device="cuda") * 1e-3).to(torch.bfloat16)

    def buffers():
        return dict(nout=torch.empty_like(state), nr=torch.empty(T, device="cuda"),
                    dw=torch.zeros(V, D, dtype=torch.float32, device="cuda"), ds=d0.clone(),
                    pp=torch.zeros(P, D, dtype=torch.float32, device="cuda"), loss=torch.empty(T, device="cuda"),
                    lse=torch.empty(T, device="cuda"))

    def call(o, stream):
        L.nm_ce_readout(1, nmce.LEV, 1, nmce.ptr(state), nmce.ptr(gain), nmce.ptr(o["nr"]), nmce.ptr(o["nout"]),
                        nmce.ptr(W), nmce.ptr(o["dw"]), nmce.ptr(o["pp"]), nmce.ptr(gs), nmce.ptr(o["ds"]), D, nmce.ptr(tg),
                        nmce.ptr(w), nmce.ptr(o["loss"]), nmce.ptr(o["lse"]), None, 0, T, D, V, chunk, EPS, nmce.ptr(ws),
                        stream)

    eager = buffers()
    call(eager, None)
    torch.cuda.synchronize()
    captured = buffers()
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        call(captured, s.cuda_stream)
    for _ in range(2):                      # replayed twice from the same starting values
        captured["dw"].zero_()
        captured["ds"].copy_(d0)
        graph.replay()
    torch.cuda.synchronize()
    for k in ("loss", "lse", "dw", "ds", "pp", "nr"):
        assert same_bits(captured[k], eager[k]), f"graph replay differs from the eager call: {k}"
    word = ctypes.c_uint32(1)
    assert L.nm_norm_bwd_device_status(None, ctypes.byref(word)) == 0 and word.value == 0

"""Bit parity of the norm backward kernels (levanter rounding) with the numpy restatement of the reference's rounding
points (oracle/ew_oracle.py). The operands that enter the row sums are drawn from small dyadic grids, so that every
partial sum is exact in f32 and the sums do not depend on the order of addition; everything else (the saved statistics,
the residual gradients) is arbitrary. dx / dx_in must then match bit for bit; the gain-gradient partials are sums of
per-row bf16 terms over the rows of a part (f32, order fixed by the kernel's geometry) and are compared with the float64
sum of the oracle's terms; the post-norm branch gradient depends on a row sum whose summands are not on a grid and is
allowed one bf16 step on a small fraction of elements. Also: the status word of the kernels' bounded waits stays 0."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
EPS = 1e-5


def _grid(rng, shape, steps, scale):
    """bf16-exact values k * scale, k in [-steps, steps]"""
    return (rng.integers(-steps, steps + 1, size=shape).astype(np.float32) * np.float32(scale))


def _dev(a, dtype=torch.bfloat16):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dtype)


def _bits(t):
    return t.view(torch.int16).cpu().numpy()


def _bits_of(a):
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16).view(np.int16)


def _part_sums(gc, parts):
    T = gc.shape[0]
    return np.stack([gc[p * T // parts:(p + 1) * T // parts].sum(0, dtype=np.float64) for p in range(parts)])


def _status_is_zero(L):
    word = ctypes.c_uint32(77)
    assert L.nm_norm_bwd_device_status(None, ctypes.byref(word)) == 0 and word.value == 0


@pytest.mark.parametrize("T,D", [(777, 2048), (300, 512), (1500, 1024), (129, 136), (64, 256), (210, 4096), (97, 8192),
                                 (40, 4104), (1, 512), (7, 2048), (5000, 8)])
@pytest.mark.parametrize("with_res", [True, False])
def test_rmsnorm_bwd_bits(T, D, with_res):
    from gpu_common import lib, nmce
    import ew_oracle
    rng = np.random.default_rng(T + D)
    x = _grid(rng, (T, D), 8, 0.25)
    dy = _grid(rng, (T, D), 8, 2.0 ** -10)
    gain = _grid(rng, (D,), 2, 0.5) + np.float32(1.5)          # 0.5 .. 2.5 in steps of 0.5
    rstd = (1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(1) + EPS) * rng.uniform(0.9, 1.1, T)).astype(np.float32)
    dres = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2) if with_res else None
    want_dx, gc = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, gain, rstd, dres, EPS)
    L = lib()
    P = int(L.nm_norm_partial_rows(T))
    dx = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    part = torch.full((P, D), float("nan"), device="cuda")
    d_dy, d_x, d_g, d_r = _dev(dy), _dev(x), _dev(gain), _dev(rstd, torch.float32)
    d_res = _dev(dres) if with_res else None
    L.nm_rmsnorm_bwd_add_partial(1, 0, nmce.ptr(d_dy), nmce.ptr(d_x), nmce.ptr(d_g), nmce.ptr(d_r), nmce.ptr(d_res),
                                 nmce.ptr(dx), nmce.ptr(part), T, D, EPS, None)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(dx), _bits_of(want_dx))
    np.testing.assert_allclose(part.cpu().numpy(), _part_sums(gc, P), rtol=2e-5, atol=1e-7)
    if with_res:   # in place over the residual gradient: same bits
        L.nm_rmsnorm_bwd_add_partial(1, 0, nmce.ptr(d_dy), nmce.ptr(d_x), nmce.ptr(d_g), nmce.ptr(d_r), nmce.ptr(d_res),
                                     nmce.ptr(d_res), None, T, D, EPS, None)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(d_res), _bits_of(want_dx))
    _status_is_zero(L)


@pytest.mark.parametrize("T,D", [(777, 2048), (300, 512), (1500, 1024), (129, 136), (64, 256), (210, 4096), (97, 8192),
                                 (1, 512), (7, 2048)])
@pytest.mark.parametrize("post", [True, False])
def test_sandwich_bwd_bits(T, D, post):
    from gpu_common import lib, nmce
    import ew_oracle
    rng = np.random.default_rng(3 * T + D + int(post))
    xo = _grid(rng, (T, D), 8, 0.25)
    b = _grid(rng, (T, D), 8, 0.25)
    da = _grid(rng, (T, D), 8, 2.0 ** -10)
    gn = _grid(rng, (D,), 2, 0.5) + np.float32(1.5)
    gp = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32)) if post else None
    dxo = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1e-2)
    rn = (1.0 / np.sqrt((xo.astype(np.float64) ** 2).mean(1) + EPS) * rng.uniform(0.9, 1.1, T)).astype(np.float32)
    rp = (1.0 / np.sqrt((b.astype(np.float64) ** 2).mean(1) + EPS) * rng.uniform(0.9, 1.1, T)).astype(np.float32)
    want_in, want_br, gcn, gcp, _ = ew_oracle.sandwich_bwd_levanter(dxo, da, xo, gn, rn, b if post else None, gp,
                                                                    rp if post else None, EPS)
    L = lib()
    P = int(L.nm_norm_partial_rows(T))
    dx_in = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    dbr = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    pgn = torch.full((P, D), float("nan"), device="cuda")
    pgp = torch.full((P, D), float("nan"), device="cuda")
    d = dict(dxo=_dev(dxo), da=_dev(da), xo=_dev(xo), gn=_dev(gn), rn=_dev(rn, torch.float32), b=_dev(b),
             gp=_dev(gp) if post else None, rp=_dev(rp, torch.float32) if post else None)
    p = nmce.ptr
    L.nm_sandwich_tail_bwd_partial(1, 0, p(d["dxo"]), p(d["da"]), p(d["xo"]), p(d["gn"]), p(d["rn"]), p(d["b"]),
                                   p(d["gp"]), p(d["rp"]), p(dx_in), p(dbr), p(pgn), p(pgp) if post else None, T, D,
                                   EPS, None)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(dx_in), _bits_of(want_in))
    np.testing.assert_allclose(pgn.cpu().numpy(), _part_sums(gcn, P), rtol=2e-5, atol=1e-7)
    if post:
        got, want = _bits(dbr).astype(np.int32), _bits_of(want_br).astype(np.int32)
        off = got != want
        assert off.mean() < 5e-3 and (np.abs(got - want)[off] <= 1).all()
        # the gain terms of the post-norm are functions of dx_mid, the branch and the saved statistic only: exact terms
        np.testing.assert_allclose(pgp.cpu().numpy(), _part_sums(gcp, P), rtol=2e-5, atol=1e-7)
    else:
        assert np.array_equal(_bits(dbr), _bits_of(want_in))
    _status_is_zero(L)


def _true_rstd(v):
    return 1.0 / np.sqrt((v.astype(np.float64) ** 2).mean(1) + EPS)


@pytest.mark.parametrize("T,D", [(777, 2048), (300, 512), (1500, 1024), (129, 136), (64, 256), (210, 4096), (97, 8192)])
def test_rmsnorm_fwd_bits(T, D):
    from gpu_common import lib, nmce
    import ew_oracle
    rng = np.random.default_rng(7 * T + D)
    x = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 2)
    gain = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    L = lib()
    d_x, d_g = _dev(x), _dev(gain)
    y = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    rstd = torch.empty(T, device="cuda")
    L.nm_rmsnorm_fwd(1, 0, nmce.ptr(d_x), nmce.ptr(d_g), nmce.ptr(y), nmce.ptr(rstd), T, D, EPS, None)
    torch.cuda.synchronize()
    r = rstd.cpu().numpy()
    np.testing.assert_allclose(r, _true_rstd(x), rtol=1e-6)       # f32 sum of 8192 squares + rsqrtf
    assert np.array_equal(_bits(y), _bits_of(ew_oracle.rmsnorm_fwd_levanter(x, gain, r)))
    # statistics only (no output): same r
    rstd2 = torch.empty(T, device="cuda")
    L.nm_rmsnorm_fwd(1, 0, nmce.ptr(d_x), nmce.ptr(d_g), None, nmce.ptr(rstd2), T, D, EPS, None)
    torch.cuda.synchronize()
    assert torch.equal(rstd, rstd2)
    _status_is_zero(L)


@pytest.mark.parametrize("T,D", [(777, 2048), (300, 512), (1500, 1024), (129, 136), (64, 256), (210, 4096), (97, 8192)])
@pytest.mark.parametrize("post", [True, False])
def test_sandwich_fwd_bits(T, D, post):
    from gpu_common import lib, nmce
    import ew_oracle
    rng = np.random.default_rng(11 * T + D + int(post))
    branch = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * 1.5)
    x_in = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32))
    gp = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32)) if post else None
    gn = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    L = lib()
    d_b, d_x, d_gn = _dev(branch), _dev(x_in), _dev(gn)
    d_gp = _dev(gp) if post else None
    x_out = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    a_next = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    rp = torch.zeros(T, device="cuda")
    rn = torch.zeros(T, device="cuda")
    p = nmce.ptr
    L.nm_sandwich_tail_fwd(1, 0, p(d_b), p(d_x), p(d_gp), p(d_gn), p(x_out), p(a_next), p(rp) if post else None, p(rn),
                           T, D, EPS, None)
    torch.cuda.synchronize()
    r_p, r_n = rp.cpu().numpy(), rn.cpu().numpy()
    if post:
        np.testing.assert_allclose(r_p, _true_rstd(branch), rtol=1e-6)
    want_xo, want_an = ew_oracle.sandwich_fwd_levanter(branch, x_in, gp, gn, r_p if post else None, r_n)
    assert np.array_equal(_bits(x_out), _bits_of(want_xo))
    np.testing.assert_allclose(r_n, _true_rstd(want_xo), rtol=1e-6)   # statistics of the stored (rounded) x_out
    assert np.array_equal(_bits(a_next), _bits_of(want_an))
    # in place over the residual stream (x_out == x_in): same bits
    inpl = d_x.clone()
    an2 = torch.empty_like(a_next)
    L.nm_sandwich_tail_fwd(1, 0, p(d_b), p(inpl), p(d_gp), p(d_gn), p(inpl), p(an2), None, None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert torch.equal(inpl, x_out) and torch.equal(an2, a_next)
    _status_is_zero(L)


def test_norm_kernels_reject_rows_longer_than_8192():
    from gpu_common import lib, nmce
    L = lib()
    T, D = 4, 8200
    a = torch.zeros(T, D, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(T, device="cuda")
    p = nmce.ptr
    raw = L.raw   # status codes instead of exceptions
    assert raw("nm_rmsnorm_fwd")(1, 0, p(a), p(g), p(a), p(r), T, D, EPS, None) == 1
    assert raw("nm_rmsnorm_bwd_add_partial")(1, 0, p(a), p(a), p(g), p(r), None, p(a), None, T, D, EPS, None) == 1
    assert raw("nm_sandwich_tail_fwd")(1, 0, p(a), p(a), None, p(g), p(a), p(a), None, p(r), T, D, EPS, None) == 1
    assert raw("nm_sandwich_tail_bwd_partial")(1, 0, p(a), p(a), p(a), p(g), p(r), p(a), None, None, p(a), p(a), None,
                                               None, T, D, EPS, None) == 1
    assert b"8192" in raw("nm_last_error")()


# ----------------------------------------------------------------------------- against the reference's own emulation
def _golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "norm_golden.npz"))


def _dev_bits(bits):
    """uint16 bf16 bit patterns -> bf16 device tensor"""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def _u16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("name", ["n512", "n136", "n2048"])
def test_rmsnorm_pair_equals_reference_emulation(name):
    """Inputs and outputs of the reference's tests/s3/levemu.py (tests/golden/norm_golden.npz): exact-sum inputs, so the
    kernels must reproduce every bit of out, dx and bf16(dres + dx); the saved statistics are the emulation's."""
    from gpu_common import lib, nmce
    G = _golden()
    eps = float(G["eps"])
    x, dy, g, dres = (_dev_bits(G[f"{name}.{k}"]) for k in ("x", "dy", "g", "dres"))
    r_emu = G[f"{name}.rstd"]
    T, D = x.shape
    L = lib()
    p = nmce.ptr
    y = torch.empty_like(x)
    rstd = torch.empty(T, device="cuda")
    L.nm_rmsnorm_fwd(1, 0, p(x), p(g), p(y), p(rstd), T, D, eps, None)
    torch.cuda.synchronize()
    np.testing.assert_allclose(rstd.cpu().numpy(), r_emu, rtol=3e-7)     # rsqrtf against torch's CPU rsqrt
    r_dev = torch.from_numpy(r_emu).cuda()
    if np.array_equal(rstd.cpu().numpy(), r_emu):
        assert np.array_equal(_u16(y), G[f"{name}.out"])
    for res, key in ((None, "dx"), (dres, "dx_res")):
        dx = torch.empty_like(x)
        part = torch.zeros(int(L.nm_norm_partial_rows(T)), D, device="cuda")
        L.nm_rmsnorm_bwd_add_partial(1, 0, p(dy), p(x), p(g), p(r_dev), p(res), p(dx), p(part), T, D, eps, None)
        torch.cuda.synchronize()
        assert np.array_equal(_u16(dx), G[f"{name}.{key}"])
        want = (G[f"{name}.dgc"].astype(np.uint32) << 16).view(np.float32).sum(0, dtype=np.float64)
        np.testing.assert_allclose(part.sum(0).cpu().numpy(), want, rtol=2e-5, atol=1e-7)
    _status_is_zero(L)


@pytest.mark.parametrize("name,post", [("s512p", True), ("s512", False), ("s136p", True), ("s2048p", True)])
def test_sandwich_equals_reference_emulation(name, post):
    from gpu_common import lib, nmce
    G = _golden()
    eps = float(G["eps"])
    b, xi, gn, dan, dxo = (_dev_bits(G[f"{name}.{k}"]) for k in ("b", "xi", "gn", "dan", "dxo"))
    gp = _dev_bits(G[f"{name}.gp"]) if post else None
    rn = torch.from_numpy(G[f"{name}.rn"]).cuda()
    rp = torch.from_numpy(G[f"{name}.rp"]).cuda() if post else None
    T, D = b.shape
    L = lib()
    p = nmce.ptr
    x_out, a_next = torch.empty_like(b), torch.empty_like(b)
    rp_k, rn_k = torch.zeros(T, device="cuda"), torch.zeros(T, device="cuda")
    L.nm_sandwich_tail_fwd(1, 0, p(b), p(xi), p(gp), p(gn), p(x_out), p(a_next), p(rp_k) if post else None, p(rn_k), T, D,
                           eps, None)
    torch.cuda.synchronize()
    np.testing.assert_allclose(rn_k.cpu().numpy(), G[f"{name}.rn"], rtol=3e-7)
    if post:
        np.testing.assert_allclose(rp_k.cpu().numpy(), G[f"{name}.rp"], rtol=3e-7)
    if not post or np.array_equal(rp_k.cpu().numpy(), G[f"{name}.rp"]):
        assert np.array_equal(_u16(x_out), G[f"{name}.x_out"])
    # the backward from the emulation's stored x_out and statistics
    xo = _dev_bits(G[f"{name}.x_out"])
    dx_in, dbr = torch.empty_like(b), torch.empty_like(b)
    P = int(L.nm_norm_partial_rows(T))
    pgn, pgp = torch.zeros(P, D, device="cuda"), torch.zeros(P, D, device="cuda")
    L.nm_sandwich_tail_bwd_partial(1, 0, p(dxo), p(dan), p(xo), p(gn), p(rn), p(b), p(gp), p(rp), p(dx_in), p(dbr), p(pgn),
                                   p(pgp) if post else None, T, D, eps, None)
    torch.cuda.synchronize()
    assert np.array_equal(_u16(dx_in), G[f"{name}.dx_in"])
    want = (G[f"{name}.dgcn"].astype(np.uint32) << 16).view(np.float32).sum(0, dtype=np.float64)
    np.testing.assert_allclose(pgn.sum(0).cpu().numpy(), want, rtol=2e-5, atol=1e-7)
    if post:
        got, ref = _u16(dbr).astype(np.int32), G[f"{name}.dbranch"].astype(np.int32)
        off = got != ref
        assert off.mean() < 5e-3 and (np.abs(got - ref)[off] <= 1).all()
    else:
        assert np.array_equal(_u16(dbr), G[f"{name}.dx_in"])
    _status_is_zero(L)


# ----------------------------------------------------------------------------- the reference's other two acceptance rules
def _rel64(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300)


@pytest.mark.parametrize("D", [512, 2048])
def test_rmsnorm_realistic_inputs_levanter_and_accurate(D):
    """The reference's rules for realistic inputs (tests/s3/test_rmsnorm.py:6-14): levanter mode equals the emulation
    bitwise on >= 99.99 % of elements (a different f32 summation order may flip rare bf16 roundings) and is no further
    from float64 than 1.25 x the emulation; accurate mode (f32 inside, one rounding per stored output) stays within
    1.05 x the error of a single bf16 rounding of the float64 result."""
    from gpu_common import lib, nmce
    import ew_oracle
    T = 2048
    rng = np.random.default_rng(D)
    x = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32) * rng.uniform(0.5, 2.0, (T, 1)).astype(np.float32))
    dy = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32))
    dres = ew_oracle.bf(rng.standard_normal((T, D)).astype(np.float32))
    g = ew_oracle.bf((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    x64, dy64, g64 = x.astype(np.float64), dy.astype(np.float64), g.astype(np.float64)
    r64 = 1.0 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + EPS)
    a64 = g64[None, :] * dy64
    out64 = g64[None, :] * x64 * r64
    dx64 = a64 * r64 - x64 * r64 ** 3 * (x64 * a64).sum(1, keepdims=True) / D + dres
    L = lib()
    p = nmce.ptr
    d_x, d_dy, d_g, d_res = _dev(x), _dev(dy), _dev(g), _dev(dres)
    for rounding in (0, 1):
        y = torch.empty_like(d_x)
        dx = torch.empty_like(d_x)
        rstd = torch.empty(T, device="cuda")
        L.nm_rmsnorm_fwd(1, rounding, p(d_x), p(d_g), p(y), p(rstd), T, D, EPS, None)
        L.nm_rmsnorm_bwd_add_partial(1, rounding, p(d_dy), p(d_x), p(d_g), p(rstd), p(d_res), p(dx), None, T, D, EPS, None)
        torch.cuda.synchronize()
        yk, dxk = y.float().cpu().numpy(), dx.float().cpu().numpy()
        if rounding == 0:
            r = rstd.cpu().numpy()
            emu_dx, _ = ew_oracle.rmsnorm_bwd_add_levanter(dy, x, g, r, dres, EPS)
            assert np.array_equal(_bits(y), _bits_of(ew_oracle.rmsnorm_fwd_levanter(x, g, r)))
            # the restatement takes its row sums in float64; the kernel in f32: only the sum's last bit may differ
            assert (_bits(dx) == _bits_of(emu_dx)).mean() >= 0.9999
            assert _rel64(dxk, dx64) <= 1.25 * _rel64(emu_dx, dx64) + 1e-12
        else:
            floor_y = _rel64(ew_oracle.bf(out64.astype(np.float32)), out64)
            floor_dx = _rel64(ew_oracle.bf(dx64.astype(np.float32)), dx64)
            assert _rel64(yk, out64) <= 1.05 * floor_y and _rel64(dxk, dx64) <= 1.05 * floor_dx
            np.testing.assert_allclose(rstd.cpu().numpy(), r64[:, 0], rtol=1e-6)
    _status_is_zero(L)


def test_norm_status_word_reports_an_expired_wait():
    """A wait of the batch ring that ran out would leave a bit in the per-GPU status word; nm_norm_bwd_device_status must
    report it once and clear it. The bit is produced the safe way: the millisecond wait probe pointed at that word (no
    norm kernel is made to wait)."""
    from gpu_common import lib, nmce
    L = lib()
    _status_is_zero(L)
    L.nm_norm_bwd_test_timeout(1_000_000, None)
    word = ctypes.c_uint32(0)
    with pytest.raises(nmce.NmError) as e:
        L.nm_norm_bwd_device_status(None, ctypes.byref(word))
    assert e.value.status == 2 and word.value == 4
    _status_is_zero(L)      # cleared by the read
    T, D = 64, 512          # and the kernels run as before
    a = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    g = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(a)
    r = torch.empty(T, device="cuda")
    L.nm_rmsnorm_fwd(1, 0, nmce.ptr(a), nmce.ptr(g), nmce.ptr(y), nmce.ptr(r), T, D, EPS, None)
    torch.cuda.synchronize()
    _status_is_zero(L)


# ----------------------------------------------------------------------------- f32 storage (math against float64)
def _norm64(x, g):
    return x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + EPS) * g


@pytest.mark.parametrize("D", [512, 136, 2048])
@pytest.mark.parametrize("post", [True, False])
def test_f32_storage_norm_kernels_against_float64(D, post):
    """The f32-storage instantiations (storage 0): f32 throughout, so every output is held to 1e-6 of float64 autograd
    (the reference's bound for them, tests/s3/test_rmsnorm.py:4), with both rounding arguments."""
    from gpu_common import lib, nmce, rel
    T = 333
    g = torch.Generator(device="cuda").manual_seed(D + int(post))
    rnd = lambda *s, k=1.0: (torch.randn(*s, generator=g, device="cuda") * k).float()
    x, b = rnd(T, D, k=2.0), rnd(T, D, k=1.5)
    gn, gp = 1.0 + 0.2 * rnd(D), (1.0 + 0.2 * rnd(D)) if post else None
    dy, dres, dxo = rnd(T, D, k=1e-2), rnd(T, D, k=1e-2), rnd(T, D, k=1e-2)
    L = lib()
    p = nmce.ptr
    P = int(L.nm_norm_partial_rows(T))
    # RMSNorm pair
    x64, g64 = x.double().requires_grad_(True), gn.double().requires_grad_(True)
    o64 = _norm64(x64, g64)
    o64.backward(dy.double())
    for rounding in (0, 1):
        y, rstd, dx = torch.empty_like(x), torch.empty(T, device="cuda"), torch.empty_like(x)
        dg = torch.zeros(D, device="cuda")
        L.nm_rmsnorm_fwd(0, rounding, p(x), p(gn), p(y), p(rstd), T, D, EPS, None)
        L.nm_rmsnorm_bwd_add(0, rounding, p(dy), p(x), p(gn), p(rstd), p(dres), p(dx), p(dg), T, D, EPS, None)
        torch.cuda.synchronize()
        assert rel(y, o64.detach()) < 1e-6 and rel(dx, x64.grad + dres.double()) < 1e-6 and rel(dg, g64.grad) < 1e-6
        assert rel(rstd, torch.rsqrt((x.double() ** 2).mean(1) + EPS)) < 1e-6
        part = torch.zeros(P, D, device="cuda")
        inpl = dres.clone()     # in place over the residual gradient, statistics recomputed (rstd = NULL)
        L.nm_rmsnorm_bwd_add_partial(0, rounding, p(dy), p(x), p(gn), None, p(inpl), p(inpl), p(part), T, D, EPS, None)
        torch.cuda.synchronize()
        assert rel(inpl, x64.grad + dres.double()) < 1e-6 and rel(part.sum(0), g64.grad) < 1e-6
    # sandwich tail
    b64, xi64 = b.double().requires_grad_(True), x.double().requires_grad_(True)
    gp64 = gp.double().requires_grad_(True) if post else None
    gn64 = gn.double().requires_grad_(True)
    xo64 = xi64 + (_norm64(b64, gp64) if post else b64)
    an64 = _norm64(xo64, gn64)
    ((an64 * dy.double()).sum() + (xo64 * dxo.double()).sum()).backward()
    x_out, a_next, dx_in, dbr = (torch.empty_like(x) for _ in range(4))
    rp, rn = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    dgn, dgp = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    L.nm_sandwich_tail_fwd(0, 0, p(b), p(x), p(gp), p(gn), p(x_out), p(a_next), p(rp) if post else None, p(rn), T, D, EPS, None)
    L.nm_sandwich_tail_bwd(0, 0, p(dxo), p(dy), p(x_out), p(gn), p(rn), p(b), p(gp), p(rp) if post else None, p(dx_in),
                           p(dbr), p(dgn), p(dgp) if post else None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert rel(x_out, xo64.detach()) < 1e-6 and rel(a_next, an64.detach()) < 1e-6
    assert rel(dx_in, xi64.grad) < 2e-6 and rel(dbr, b64.grad) < 2e-6 and rel(dgn, gn64.grad) < 2e-6
    if post:
        assert rel(dgp, gp64.grad) < 2e-6
    _status_is_zero(L)

"""The AdamH update of the LM head on the GPU (nm_adamh_update: the reference's one-tensor entry point; HeadAdamH:
the owned-ranges form) against the CPU oracle. What is pinned and where the bars come from:
  * one step from mu = nu = 0 at g = 0.5: mu, nu bit patterns and the kept Frobenius norm (the reference's
    tests/s6/test_engine.cpp:723-770);
  * moments bit-equal to the oracle's f32 operation order; p within rel-L2 1e-6 of the f64 update and element-wise
    within 2e-6 of the largest |p| (test_engine.cpp:503-534 holds 2e-6 per element on its data); the bf16 copy is
    exactly bf16(p);
  * a zero learning rate moves p by at most 1 ulp (tests/s6/test_t1_7.py:365-369); repeat runs are bitwise equal;
  * the head's own clip (gn = ||g||, clips unless gn < max) computed on the device;
  * the full-size head [128256, 2048] keeps its norm, and a strided subsample of mu matches the oracle."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HY = dict(eta=0.02, b1=0.9, b2=0.98, eps=1e-20)


def _A():
    import gpu_common  # noqa: F401  (puts oracle/ on the path)
    import adamh_oracle as A
    return A


def _state(seed, shape):
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    mu = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    nu = ((rng.standard_normal(shape) * 1e-3) ** 2).astype(np.float32)
    return p, g, mu, nu


def _run_one(p, g, mu, nu, t, eta=0.02, clip_gn=0.0, clip=False, max_norm=1.0, want16=True):
    from gpu_common import lib, nmce
    P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
    P16 = torch.zeros(p.shape, dtype=torch.bfloat16, device="cuda") if want16 else None
    R, C = p.shape
    lib().nm_adamh_update(nmce.ptr(P), nmce.ptr(P16), nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), R, C, t, eta, HY["b1"],
                          HY["b2"], HY["eps"], float(clip_gn), int(clip), max_norm, None, None, None, 0, None)
    torch.cuda.synchronize()
    return P, M, V, P16


def test_first_step_bits_and_norm():
    A = _A()
    rng = np.random.default_rng(1000)
    p = (rng.standard_normal((64, 64)) * 0.02).astype(np.float32)
    g = np.full((64, 64), 0.5, np.float32)
    z = np.zeros((64, 64), np.float32)
    P, M, V, _ = _run_one(p, g, z, z, 1)
    mu_want = A.one_minus(0.9) * np.float32(0.5)
    nu_want = A.one_minus(0.98) * (np.float32(0.5) * np.float32(0.5))
    assert (M.cpu().numpy().view(np.uint32) == mu_want.view(np.uint32)).all()
    assert (V.cpu().numpy().view(np.uint32) == nu_want.view(np.uint32)).all()
    n0, n1 = np.linalg.norm(p.astype(np.float64)), float(P.double().norm())
    assert abs(n1 - n0) <= 1e-6 * n0


@pytest.mark.parametrize("shape,t,clip", [((96, 64), 3, False), ((33, 7), 1, True), ((257, 40), 1000, True),
                                          ((1, 1), 2, False), ((2050, 520), 17, True)])
def test_against_the_oracle(shape, t, clip):
    A = _A()
    p, g, mu, nu = _state(sum(shape) + t, shape)
    max_norm = 1e-3 if clip else 1e9
    gn, do_clip = A.clip_state(g, max_norm)
    assert do_clip == clip
    P, M, V, P16 = _run_one(p, g, mu, nu, t, clip_gn=gn, clip=do_clip, max_norm=max_norm)
    p2, mu2, nu2, _ = A.adamh_f32(p, g, mu, nu, t, clip_gn=gn, clip=do_clip, max_norm=max_norm, **HY)
    q2, _, _ = A.adamh_f64(p, g, mu, nu, t, clip_gn=gn, clip=do_clip, max_norm=max_norm, **HY)
    assert np.array_equal(M.cpu().numpy(), mu2) and np.array_equal(V.cpu().numpy(), nu2), "moments are bit-exact"
    got = P.cpu().numpy()
    assert np.linalg.norm(got - q2) <= 1e-6 * np.linalg.norm(q2)
    assert np.abs(got - q2).max() <= 2e-6 * np.abs(q2).max()
    assert np.linalg.norm(got - p2) <= 2e-7 * np.linalg.norm(p2)          # against the f32 operation order
    assert torch.equal(P16, P.bfloat16())


def test_zero_learning_rate_and_repeat():
    p, g, mu, nu = _state(9, (300, 72))
    P, M, V, _ = _run_one(p, g, mu, nu, 4, eta=0.0)
    ulp = (P.cpu().numpy().view(np.int32).astype(np.int64) - p.view(np.int32).astype(np.int64))
    assert np.abs(ulp).max() <= 1
    a = _run_one(p, g, mu, nu, 4)
    b = _run_one(p, g, mu, nu, 4)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_bad_arguments():
    from gpu_common import lib, nmce
    x = torch.zeros(8, 8, device="cuda")
    blk = torch.full((8,), 3, dtype=torch.int32, device="cuda")
    with pytest.raises(nmce.NmError) as e:      # a block id outside [0, n_blocks)
        lib().nm_adamh_update(nmce.ptr(x), None, nmce.ptr(x), nmce.ptr(x), nmce.ptr(x), 8, 8, 1, 0.02, 0.9, 0.98, 1e-20,
                              0.0, 0, 1.0, nmce.ptr(blk), None, None, 2, None)
    assert e.value.status == 1 and "out of range" in str(e.value)
    with pytest.raises(nmce.NmError) as e:      # multipliers without a partition
        lib().nm_adamh_update(nmce.ptr(x), None, nmce.ptr(x), nmce.ptr(x), nmce.ptr(x), 8, 8, 1, 0.02, 0.9, 0.98, 1e-20,
                              0.0, 0, 1.0, None, nmce.ptr(x), None, 2, None)
    assert e.value.status == 1
    with pytest.raises(nmce.NmError) as e:
        lib().nm_adamh_update(nmce.ptr(x), None, nmce.ptr(x), nmce.ptr(x), nmce.ptr(x), 8, 8, 0, 0.02, 0.9, 0.98, 1e-20,
                              0.0, 0, 1.0, None, None, None, 0, None)
    assert e.value.status == 1


def _head(V, D, reducer=None):
    from gpu_common import lib
    h = ctypes.c_void_p()
    lib().nm_head_adamh_create(V, D, reducer, ctypes.byref(h))
    return h


@pytest.mark.parametrize("max_norm", [0.0, 0.05, 1e9])
def test_head_updater_with_device_side_clip(max_norm):
    A = _A()
    from gpu_common import lib, nmce
    V, D, t = 1000, 64, 6
    p, g, mu, nu = _state(21, (V, D))
    p = torch.from_numpy(p).bfloat16().float().numpy()           # the master copy starts as f32(bf16 replica)
    W16 = torch.from_numpy(p).cuda().bfloat16()
    G, M, Vv = (torch.from_numpy(a.copy()).cuda() for a in (g, mu, nu))
    h = _head(V, D)
    assert lib().nm_head_adamh_owned_elems(h) == V * D
    P = torch.empty(V * D, dtype=torch.float32, device="cuda")
    lib().nm_head_adamh_init_master(h, nmce.ptr(W16), nmce.ptr(P), None)
    assert torch.equal(P.view(V, D).cpu(), torch.from_numpy(p))
    lib().nm_head_adamh_step(h, t, HY["eta"], HY["b1"], HY["b2"], HY["eps"], max_norm, 1.0, nmce.ptr(G), nmce.ptr(P),
                             nmce.ptr(M), nmce.ptr(Vv), nmce.ptr(W16), None)
    sc = (ctypes.c_double * 4)()
    lib().nm_head_adamh_scalars(h, sc, None)
    if max_norm > 0:
        gn, clip = A.clip_state(g, max_norm)
        assert abs(np.sqrt(sc[0]) - gn) <= 1e-6 * gn
        assert clip == (max_norm == 0.05)
    else:
        gn, clip = 0.0, False
    p2, mu2, nu2, _ = A.adamh_f32(p, g, mu, nu, t, clip_gn=gn, clip=clip, max_norm=max_norm or 1.0, **HY)
    assert np.array_equal(M.cpu().numpy(), mu2) and np.array_equal(Vv.cpu().numpy(), nu2)
    assert np.linalg.norm(P.view(V, D).cpu().numpy() - p2) <= 2e-7 * np.linalg.norm(p2)
    assert torch.equal(W16, P.view(V, D).bfloat16())
    lib().nm_head_adamh_destroy(h)


def test_owned_ranges_through_a_one_rank_reducer():
    """Five buckets through a reducer that reduces to owners on a one-rank communicator: the multi-range walk, the
    in-place reduce-scatter and all-gather calls, against the oracle on the whole tensor."""
    A = _A()
    from gpu_common import lib, nmce
    V, D, t = 1000, 72, 3
    p, g, mu, nu = _state(33, (V, D))
    idbuf = np.zeros(128, np.uint8)
    lib().nm_comm_unique_id(nmce.ptr(idbuf))
    comm, red = ctypes.c_void_p(), ctypes.c_void_p()
    lib().nm_comm_create(nmce.ptr(idbuf), 1, 0, ctypes.byref(comm))
    G = torch.from_numpy(g.copy()).cuda()
    lib().nm_grad_reducer_create_owners(comm, nmce.ptr(G), V, D, 5, ctypes.byref(red))
    h = _head(V, D, red)
    go, co, ln, nr = (ctypes.c_int64 * 64)(), (ctypes.c_int64 * 64)(), (ctypes.c_int64 * 64)(), ctypes.c_int(0)
    lib().nm_head_adamh_ranges(h, 64, go, co, ln, ctypes.byref(nr))
    assert nr.value == 5 and go[0] == 0 and sum(ln[i] for i in range(5)) == V * D
    assert all(go[i] == co[i] for i in range(5))                 # one rank: compact = global
    P, M, Vv = (torch.from_numpy(a.copy()).cuda().view(-1) for a in (p, mu, nu))
    W16 = torch.zeros(V, D, dtype=torch.bfloat16, device="cuda")
    lib().nm_grad_reducer_reduce_all(red, None)
    lib().nm_head_adamh_step(h, t, HY["eta"], HY["b1"], HY["b2"], HY["eps"], 0.01, 1.0, nmce.ptr(G), nmce.ptr(P),
                             nmce.ptr(M), nmce.ptr(Vv), nmce.ptr(W16), None)
    torch.cuda.synchronize()
    gn, clip = A.clip_state(g, 0.01)
    p2, mu2, nu2, _ = A.adamh_f32(p, g, mu, nu, t, clip_gn=gn, clip=clip, max_norm=0.01, **HY)
    assert np.array_equal(M.view(V, D).cpu().numpy(), mu2) and np.array_equal(Vv.view(V, D).cpu().numpy(), nu2)
    assert np.linalg.norm(P.view(V, D).cpu().numpy() - p2) <= 2e-7 * np.linalg.norm(p2)
    assert torch.equal(W16, P.view(V, D).bfloat16())
    lib().nm_head_adamh_destroy(h)
    lib().nm_grad_reducer_destroy(red)
    lib().nm_comm_destroy(comm)


def test_full_size_head_keeps_its_norm():
    A = _A()
    from gpu_common import lib, nmce
    V, D, t = 128256, 2048, 11
    gen = torch.Generator(device="cuda").manual_seed(5)
    P = torch.randn(V * D, generator=gen, device="cuda") * 0.02
    G = torch.randn(V * D, generator=gen, device="cuda") * 1e-4
    M = torch.randn(V * D, generator=gen, device="cuda") * 1e-4
    Vv = (torch.randn(V * D, generator=gen, device="cuda") * 1e-4) ** 2
    W16 = torch.empty(V, D, dtype=torch.bfloat16, device="cuda")
    n0 = float(P.double().norm())
    sub = slice(12345, V * D, 1000003)
    p_s, g_s, m_s, v_s = (a[sub].cpu().numpy() for a in (P, G, M, Vv))
    gn = float(G.double().norm())
    h = _head(V, D)
    lib().nm_head_adamh_step(h, t, HY["eta"], HY["b1"], HY["b2"], HY["eps"], 0.5 * gn, 1.0, nmce.ptr(G), nmce.ptr(P),
                             nmce.ptr(M), nmce.ptr(Vv), nmce.ptr(W16), None)
    torch.cuda.synchronize()
    n1 = float(P.double().norm())
    assert abs(n1 - n0) <= 1e-6 * n0
    sc = (ctypes.c_double * 4)()
    lib().nm_head_adamh_scalars(h, sc, None)
    assert abs(np.sqrt(sc[0]) - gn) <= 1e-6 * gn and abs(np.sqrt(sc[1]) - n0) <= 1e-6 * n0
    # moments of a strided subsample, bit-exact against the oracle's element arithmetic with the device's clip norm
    F = np.float32
    gn32 = np.sqrt(F(sc[0]))
    gi = (g_s / gn32) * F(0.5 * gn)
    mu_w = A.one_minus(0.9) * gi + F(0.9) * m_s
    nu_w = A.one_minus(0.98) * (gi * gi) + F(0.98) * v_s
    assert np.array_equal(M[sub].cpu().numpy(), mu_w) and np.array_equal(Vv[sub].cpu().numpy(), nu_w)
    assert torch.equal(W16.view(-1)[sub], P[sub].bfloat16())
    lib().nm_head_adamh_destroy(h)


@pytest.mark.parametrize("shape,t,clip", [((1, 2048), 1, False), ((96, 64), 3, True), ((33, 7), 40, True)])
def test_plain_adam_is_bit_exact_against_the_oracle(shape, t, clip):
    """nm_adam_update (the rule of the final norm's gain): every operation is elementwise in the reference's order, so
    p, mu, nu are bit-equal to the oracle (the reference's own test compares bitwise with host f32,
    tests/s6/test_engine.cpp:756-761)."""
    A = _A()
    from gpu_common import lib, nmce
    p, g, mu, nu = _state(7 * sum(shape) + t, shape)
    max_norm = 1e-3 if clip else 1e9
    gn, do_clip = A.clip_state(g, max_norm)
    P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
    P16 = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    lib().nm_adam_update(nmce.ptr(P), nmce.ptr(P16), nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), shape[0], shape[1], t, 0.008,
                         0.9, 0.98, 1e-20, float(gn), int(do_clip), max_norm, None, None, None, 0, None)
    torch.cuda.synchronize()
    p2, mu2, nu2 = A.adam_f32(p, g, mu, nu, t, 0.008, 0.9, 0.98, 1e-20, clip_gn=gn, clip=do_clip, max_norm=max_norm)
    assert np.array_equal(M.cpu().numpy(), mu2) and np.array_equal(V.cpu().numpy(), nu2)
    assert np.array_equal(P.cpu().numpy(), p2)
    assert torch.equal(P16, P.bfloat16())


def test_update_stays_inside_its_buffers():
    """p, mu, nu and the bf16 copy between guard bands, with an element count that is not a multiple of 4 and buffers
    that are not 16-byte aligned (the scalar walk): nothing outside the tensor is written."""
    from gpu_common import lib, nmce
    R, C = 37, 11
    n = R * C
    p, g, mu, nu = _state(55, (R, C))
    G = 1024

    def guarded(arr, dtype, esz):
        buf = torch.full((G + 4 + n * esz + G,), 0xA5, dtype=torch.uint8, device="cuda")
        view = buf[G + 4:G + 4 + n * esz].view(dtype)          # 4 bytes past a 16-byte boundary
        if arr is not None:
            view.copy_(torch.from_numpy(arr.reshape(-1)).cuda())
        return buf, view

    bp, vp = guarded(p, torch.float32, 4)
    bm, vm = guarded(mu, torch.float32, 4)
    bv, vv = guarded(nu, torch.float32, 4)
    b16, v16 = guarded(None, torch.bfloat16, 2)
    G_ = torch.from_numpy(g.copy()).cuda()
    lib().nm_adamh_update(nmce.ptr(vp), nmce.ptr(v16), nmce.ptr(G_), nmce.ptr(vm), nmce.ptr(vv), R, C, 2, 0.02, 0.9, 0.98,
                          1e-20, 0.0, 0, 1.0, None, None, None, 0, None)
    torch.cuda.synchronize()
    for name, buf, esz in (("p", bp, 4), ("mu", bm, 4), ("nu", bv, 4), ("p16", b16, 2)):
        assert bool((buf[:G + 4] == 0xA5).all()) and bool((buf[G + 4 + n * esz:] == 0xA5).all()), f"{name}: guard written"
    assert torch.equal(v16, vp.bfloat16())
    assert abs(float(vp.double().norm()) - float(np.linalg.norm(p.astype(np.float64)))) <= 1e-6 * float(np.linalg.norm(p))


@pytest.mark.parametrize("rule", ["adam", "adamh"])
def test_row_blocks_own_rates_norms_and_frozen_rows(rule):
    """The case of the reference's engine test (tests/s6/test_engine.cpp:416-534) through the one-tensor entry points: a
    [96, 64] tensor, rows [0, 32) block 0 with learning rate x 0.5, [32, 64) block 1 frozen, [64, 96) block 2; frozen
    rows keep p, mu, nu; each AdamH block keeps its own Frobenius norm (1e-6); element error against the f64 update
    within 2e-6; against the oracle's f32 order: Adam bit-equal, AdamH 2e-7."""
    A = _A()
    from gpu_common import lib, nmce
    R, C, t = 96, 64, 1
    p, g, mu, nu = _state(100, (R, C))
    mu *= 0.1
    bor = (np.arange(R) // 32).astype(np.int32)
    mult = np.array([0.5, 0.5, 1.0], np.float32)
    frozen = np.array([0, 1, 0], np.uint8)
    lr = 0.008 if rule == "adam" else 0.02
    P, G, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, g, mu, nu))
    P16 = torch.full((R, C), 7.0, dtype=torch.bfloat16, device="cuda")
    B, MU, FR = torch.from_numpy(bor).cuda(), torch.from_numpy(mult).cuda(), torch.from_numpy(frozen).cuda()
    fn = lib().nm_adam_update if rule == "adam" else lib().nm_adamh_update
    fn(nmce.ptr(P), nmce.ptr(P16), nmce.ptr(G), nmce.ptr(M), nmce.ptr(V), R, C, t, lr, 0.9, 0.98, 1e-20, 0.0, 0, 1.0,
       nmce.ptr(B), nmce.ptr(MU), nmce.ptr(FR), 3, None)
    torch.cuda.synchronize()
    ofn = A.adam_f32 if rule == "adam" else A.adamh_f32
    p2, mu2, nu2 = A.with_row_blocks(ofn, p, g, mu, nu, t, lr, 0.9, 0.98, 1e-20, bor, mult, frozen)
    got, gm, gv = P.cpu().numpy(), M.cpu().numpy(), V.cpu().numpy()
    fr = bor == 1
    assert np.array_equal(got[fr], p[fr]) and np.array_equal(gm[fr], mu[fr]) and np.array_equal(gv[fr], nu[fr])
    assert bool((P16[32:64] == 7.0).all()) and torch.equal(P16[:32], P[:32].bfloat16()) and torch.equal(P16[64:], P[64:].bfloat16())
    assert np.array_equal(gm, mu2) and np.array_equal(gv, nu2)
    if rule == "adam":
        assert np.array_equal(got, p2)
    else:
        assert np.linalg.norm(got - p2) <= 2e-7 * np.linalg.norm(p2)
        for blk in (0, 2):
            rows = bor == blk
            n0, n1 = np.linalg.norm(p[rows].astype(np.float64)), np.linalg.norm(got[rows].astype(np.float64))
            assert abs(n1 - n0) <= 1e-6 * n0
            q2, _, _ = A.adamh_f64(p[rows], g[rows], mu[rows], nu[rows], t, np.float32(lr) * mult[blk], 0.9, 0.98, 1e-20)
            assert np.abs(got[rows] - q2).max() <= 2e-6 * np.abs(q2).max()

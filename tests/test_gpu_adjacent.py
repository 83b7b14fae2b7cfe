"""GPU parity of the kernels on either side of the fused CE: doc_meta (integer outputs, bit-exact against the numpy
oracle and the reference-made golden vectors; the case list of the reference's tests/s3/test_misc.py), the fixed-order
reductions, and the sandwich tail forward / backward against a float64 torch reference."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
EOS = 128001
EPS = 1e-5


def _run_doc_meta(tok, valid, max_segs):
    from gpu_common import lib, nmce
    rows, S = tok.shape
    t = torch.from_numpy(tok).cuda()
    v = torch.from_numpy(valid.astype(np.uint8)).cuda()
    T = rows * S
    targets = torch.empty(T, dtype=torch.int32, device="cuda")
    weight = torch.empty(T, device="cuda")
    pos = torch.empty(T, dtype=torch.int32, device="cuda")
    cu = torch.full((rows * max_segs + 1,), -1, dtype=torch.int32, device="cuda")
    nseg = torch.zeros(1, dtype=torch.int32, device="cuda")
    rss = torch.full((rows, max_segs + 1), -1, dtype=torch.int32, device="cuda")
    ovf = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib().nm_doc_meta(nmce.ptr(t), nmce.ptr(v), rows, S, EOS, max_segs, nmce.ptr(targets), nmce.ptr(weight),
                      nmce.ptr(pos), nmce.ptr(cu), nmce.ptr(nseg), nmce.ptr(rss), nmce.ptr(ovf), None)
    torch.cuda.synchronize()
    return (targets.cpu().numpy().reshape(rows, S), weight.cpu().numpy().reshape(rows, S),
            pos.cpu().numpy().reshape(rows, S), rss.cpu().numpy(), cu.cpu().numpy(), int(nseg.item()),
            bool(ovf.item()))


NAMES = ("targets", "weight", "pos", "row_seg_start", "cu_seqlens", "n_segments", "overflow")


def test_doc_meta_golden():
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ew_golden.npz"))
    got = _run_doc_meta(g["dm_tok"], g["dm_valid"], int(g["dm_max_segs"]))
    want = (g["dm_targets"], g["dm_weight"], g["dm_pos"], g["dm_rss"], g["dm_cu"], int(g["dm_n"]), bool(g["dm_overflow"]))
    for n, a, b in zip(NAMES, got, want):
        assert np.array_equal(np.asarray(a), np.asarray(b)), n


@pytest.mark.parametrize("S", [4096, 4224, 4480, 19456])
def test_doc_meta_cases(S):
    """EOS at a row start and at the last position, consecutive EOS, a boundary at a tile edge, more segments than
    max_segs (overflow), an invalid row."""
    import ew_oracle as E
    rng = np.random.default_rng(S)
    rows, max_segs = 6, 24
    tok = rng.integers(0, 128000, size=(rows, S)).astype(np.int32)
    tok[0, 0] = EOS
    tok[0, S - 1] = EOS
    tok[1, 100:103] = EOS
    tok[1, 2047] = EOS
    tok[1, 255] = EOS
    for p in rng.choice(S - 1, 30, replace=False):
        tok[3, p] = EOS
    tok[4, rng.choice(S - 1, 10, replace=False)] = EOS
    valid = np.ones(rows, bool)
    valid[5] = False
    ref = E.doc_meta(tok, valid, EOS, max_segs)
    got = _run_doc_meta(tok, valid, max_segs)
    for n, a, b in zip(NAMES, got, ref):
        assert np.array_equal(np.asarray(a), np.asarray(b)), f"S={S}: {n}"
    assert ref[6]


def test_doc_meta_many_rows_and_limits():
    import ew_oracle as E
    from gpu_common import nmce
    rng = np.random.default_rng(1)
    S, max_segs = 64, 4
    for rows in (1, 12288, 16384):
        tok = rng.integers(0, 128000, size=(rows, S)).astype(np.int32)
        tok[rng.random((rows, S)) < 0.03] = EOS
        valid = rng.random(rows) > 0.01
        ref = E.doc_meta(tok, valid, EOS, max_segs)
        got = _run_doc_meta(tok, valid, max_segs)
        for n, a, b in zip(NAMES, got, ref):
            assert np.array_equal(np.asarray(a), np.asarray(b)), f"rows={rows}: {n}"
    with pytest.raises(nmce.NmError) as e:
        _run_doc_meta(np.zeros((16385, 8), np.int32), np.ones(16385, bool), 2)
    assert "16384" in str(e.value)
    tok = rng.integers(0, 1000, size=(2, 4096)).astype(np.int32)
    got = _run_doc_meta(tok, np.ones(2, bool), 24)
    assert not got[6] and got[5] == 2


def test_sum_fixed_and_reduce_partials():
    import ew_oracle as E
    from gpu_common import lib, nmce
    rng = np.random.default_rng(2)
    out = torch.zeros(1, device="cuda")
    for n in (0, 1, 1000, 1 << 20):
        x = rng.standard_normal(n).astype(np.float32)
        xt = torch.from_numpy(x).cuda() if n else torch.zeros(1, device="cuda")
        lib().nm_sum_fixed(nmce.ptr(xt), n, nmce.ptr(out), None)
        torch.cuda.synchronize()
        assert np.float32(out.item()) == E.sum_fixed(x), f"sum_fixed bits, n={n}"
    for nb, w in ((1, 64), (7, 100), (1024, 2048), (257, 512)):
        p = rng.standard_normal((nb, w)).astype(np.float32)
        out0 = rng.standard_normal(w).astype(np.float32)
        ref = p.astype(np.float64).sum(0)
        pt = torch.from_numpy(p).cuda()
        for acc in (0, 1):
            for rbf in (0, 1):
                o = torch.from_numpy(out0.copy()).cuda()
                lib().nm_reduce_partials_rows(nmce.ptr(pt), nb, w, nmce.ptr(o), acc, rbf, None)
                torch.cuda.synchronize()
                got = o.cpu().numpy().astype(np.float64) - (out0 if acc else 0)
                r = np.linalg.norm(got - ref) / np.linalg.norm(ref)
                assert r <= (4e-3 if rbf else 1e-6), f"nb={nb} w={w} acc={acc} round={rbf}: rel {r:.2e}"
                if rbf and not acc:
                    assert ((o.cpu().numpy().view(np.uint32) & 0xFFFF) == 0).all()


def _norm64(x, g):
    return x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + EPS) * g


@pytest.mark.parametrize("D", [512, 2048, 136])
@pytest.mark.parametrize("rounding", [0, 1])
@pytest.mark.parametrize("post", [True, False])
def test_sandwich_tail_against_float64(D, rounding, post):
    from gpu_common import lib, nmce, rel
    T = 700
    g = torch.Generator(device="cuda").manual_seed(D + rounding)
    bf = torch.bfloat16
    branch = (torch.randn(T, D, generator=g, device="cuda") * 1.5).to(bf)
    x_in = torch.randn(T, D, generator=g, device="cuda").to(bf)
    gp = (1.0 + 0.2 * torch.randn(D, generator=g, device="cuda")).to(bf) if post else None
    gn = (1.0 + 0.2 * torch.randn(D, generator=g, device="cuda")).to(bf)
    x_out = torch.empty_like(x_in)
    a_next = torch.empty_like(x_in)
    rp = torch.empty(T, device="cuda")
    rn = torch.empty(T, device="cuda")
    L = lib()
    L.nm_sandwich_tail_fwd(1, rounding, nmce.ptr(branch), nmce.ptr(x_in), nmce.ptr(gp), nmce.ptr(gn), nmce.ptr(x_out),
                           nmce.ptr(a_next), nmce.ptr(rp) if post else None, nmce.ptr(rn), T, D, EPS, None)
    b64 = branch.double().requires_grad_(True)
    xi64 = x_in.double().requires_grad_(True)
    gp64 = gp.double().requires_grad_(True) if post else None
    gn64 = gn.double().requires_grad_(True)
    y64 = _norm64(b64, gp64) if post else b64
    xo64 = xi64 + y64
    an64 = _norm64(xo64, gn64)
    torch.cuda.synchronize()
    assert rel(x_out, xo64) < 4e-3 and rel(a_next, an64) < 6e-3
    assert rel(rn, torch.rsqrt((x_out.double() ** 2).mean(1) + EPS)) < 1e-6     # rstd of the stored (rounded) x_out
    da = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    dxo = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    (an64 * da.double()).sum().backward(retain_graph=True)
    (xo64 * dxo.double()).sum().backward()
    dx_in = torch.empty_like(x_in)
    dbranch = torch.empty_like(x_in)
    dgn = torch.zeros(D, device="cuda")
    dgp = torch.zeros(D, device="cuda")
    L.nm_sandwich_tail_bwd(1, rounding, nmce.ptr(dxo), nmce.ptr(da), nmce.ptr(x_out), nmce.ptr(gn), nmce.ptr(rn),
                           nmce.ptr(branch), nmce.ptr(gp), nmce.ptr(rp) if post else None, nmce.ptr(dx_in),
                           nmce.ptr(dbranch), nmce.ptr(dgn), nmce.ptr(dgp) if post else None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert rel(dx_in, xi64.grad) < 8e-3
    assert rel(dbranch, b64.grad) < 1.2e-2
    assert rel(dgn, gn64.grad) < 1e-2
    if post:
        assert rel(dgp, gp64.grad) < 1.2e-2
    # in place over the residual gradient (dx_in == dx_out) gives the same bits
    inpl = dxo.clone()
    db2 = torch.empty_like(x_in)
    L.nm_sandwich_tail_bwd(1, rounding, nmce.ptr(inpl), nmce.ptr(da), nmce.ptr(x_out), nmce.ptr(gn), nmce.ptr(rn),
                           nmce.ptr(branch), nmce.ptr(gp), nmce.ptr(rp) if post else None, nmce.ptr(inpl),
                           nmce.ptr(db2), None, None, T, D, EPS, None)
    torch.cuda.synchronize()
    assert torch.equal(inpl, dx_in) and torch.equal(db2, dbranch)


def test_rmsnorm_bwd_add_reduced_gain_gradient():
    from gpu_common import lib, nmce, rel
    T, D = 1500, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    bf = torch.bfloat16
    x = (torch.randn(T, D, generator=g, device="cuda") * 2).to(bf)
    gain = (1.0 + 0.2 * torch.randn(D, generator=g, device="cuda")).to(bf)
    dy = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    x64 = x.double().requires_grad_(True)
    g64 = gain.double().requires_grad_(True)
    (_norm64(x64, g64) * dy.double()).sum().backward()
    for rounding in (0, 1):
        dx = torch.empty_like(x)
        dgain = torch.zeros(D, device="cuda")
        lib().nm_rmsnorm_bwd_add(1, rounding, nmce.ptr(dy), nmce.ptr(x), nmce.ptr(gain), None, None, nmce.ptr(dx),
                                 nmce.ptr(dgain), T, D, EPS, None)
        torch.cuda.synchronize()
        assert rel(dx, x64.grad) < 6e-3 and rel(dgain, g64.grad) < 6e-3
        if rounding == 0:   # levanter: the reduced gain gradient is a bf16 value
            assert ((dgain.cpu().numpy().view(np.uint32) & 0xFFFF) == 0).all()

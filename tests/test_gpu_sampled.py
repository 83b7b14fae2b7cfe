"""The sampled-softmax head (nm_ce_sampled_head) against its float64 oracle: the candidate list must be the oracle's to
the element; loss and lse within 2e-5, dX and dW within 3e-3 relative with cosine >= 0.9999 (the parity bars of the
full head); rows of dW outside the candidate set must keep their bits. With enough negatives to cover the whole
vocabulary the head must reproduce the full head bit for bit."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(X, W, Y, WT, gs, n_neg, offset, p_max, chunk, dw=None, z_loss=0.0, ignore_index=-(2 ** 31), fwd=False, store=1):
    from gpu_common import lib, nmce
    T, D = X.shape
    V = W.shape[0]
    ws = torch.empty(lib().nm_ce_sampled_workspace_bytes(T, D, V, p_max, chunk, store), dtype=torch.uint8, device="cuda")
    loss = torch.full((T,), float("nan"), device="cuda")
    lse = torch.full((T,), float("nan"), device="cuda")
    lp = torch.empty((T + chunk - 1) // chunk, device="cuda")
    dx = None if fwd else torch.empty_like(X)
    if dw is None and not fwd:
        dw = torch.zeros(V, D, device="cuda")
    cand = torch.full((p_max,), -7, dtype=torch.int32, device="cuda")
    n = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib().nm_ce_sampled_head(1, store, nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT), nmce.ptr(gs), nmce.ptr(loss),
                             nmce.ptr(lse), nmce.ptr(lp), nmce.ptr(dx), 0, nmce.ptr(dw), int(fwd), T, D, V, n_neg, offset,
                             p_max, chunk, nmce.ptr(cand), nmce.ptr(n), nmce.ptr(ws), None, float(z_loss),
                             int(ignore_index))
    torch.cuda.synchronize()
    # the CE workspace is the last region of the sampled head's workspace; its status word must be clean
    return loss, lse, dx, dw, lp, cand, int(n.item())


@pytest.mark.parametrize("T,D,V,n_neg,chunk,z_loss", [
    (700, 256, 5000, 512, 256, 0.0),
    (1300, 136, 1003, 100, 1024, 1e-3),          # ragged vocabulary and hidden size; nearly every id is a candidate
    (16384, 512, 128256, 16384, 16384, 1e-4),    # one readout of config 4 with as many negatives as rows
])
def test_sampled_head_matches_the_oracle(T, D, V, n_neg, chunk, z_loss):
    import sampled_oracle as S
    from gpu_common import GRAD_COS, GRAD_REL, LOSS_TOK, O, cos, grad_scale_dev, rel, to_dev
    x, w, y, wt = O.make_inputs(T, D, V, seed=T + V, ignore_frac=0.05, labels="zipf")
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    p_max = (min(V, T + n_neg) + 7) // 8 * 8
    g = torch.Generator(device="cuda").manual_seed(3)
    before = torch.randn(V, D, generator=g, device="cuda") * 1e-3
    dw = before.clone()
    offset = 987654321012
    loss, lse, dx, dw, lp, cand, n = _call(X, W, Y, WT, gs, n_neg, offset, p_max, chunk, dw=dw, z_loss=z_loss)
    ol, olse, odx, odw, ocand = S.sampled_ce_f64(x, w, y, wt, float(gs.item()), n_neg, offset, z_loss=z_loss)
    assert n == ocand.size
    assert np.array_equal(cand[:n].cpu().numpy(), ocand), "candidate list differs from the oracle's"
    assert bool((cand[n:] == -1).all())
    assert np.abs(loss.cpu().numpy() - ol).max() <= LOSS_TOK and np.abs(lse.cpu().numpy() - olse).max() <= LOSS_TOK
    got_dw = (dw - before).cpu().numpy()
    rx, rw = rel(dx, odx), rel(got_dw, odw)
    print(f"[parity] sampled head T{T} D{D} V{V} |C|={n}: loss {np.abs(loss.cpu().numpy() - ol).max():.2e} "
          f"dX rel {rx:.2e} dW rel {rw:.2e}")
    assert rx <= GRAD_REL and cos(dx, odx) >= GRAD_COS
    # dW: the update is formed in f32 on top of the previous content, so compare after subtracting it, with the bar
    # widened by the rounding of that subtraction (|before| ~ 1e-3 against updates of ~1e-5 .. 1e-3)
    assert rw <= GRAD_REL + 1e-3 and cos(got_dw, odw) >= GRAD_COS - 1e-4
    outside = np.setdiff1d(np.arange(V), ocand)
    if outside.size:
        idx = torch.from_numpy(outside).cuda()
        assert torch.equal(dw[idx], before[idx]), "a row outside the candidate set was touched"
    assert abs(float(lp.double().sum()) - float((loss.double() * WT).sum())) <= 1e-6 * abs(float(lp.double().sum()))


def test_all_ids_as_candidates_reproduce_the_full_head():
    """Negatives that cover the vocabulary (the stride is coprime with V) make C = [0, V): W_P = W, and every output
    must carry the bits of the full head."""
    from gpu_common import O, grad_scale_dev, run_ce, same_bits, to_dev
    T, D, V, chunk = 1500, 512, 8256, 512
    x, w, y, wt = O.make_inputs(T, D, V, seed=6, ignore_frac=0.05)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    full = run_ce(X, W, Y, WT, gs, chunk=chunk, z_loss=1e-4)
    loss, lse, dx, dw, lp, cand, n = _call(X, W, Y, WT, gs, V, 5, V, chunk, z_loss=1e-4)
    assert n == V and bool((cand.cpu() == torch.arange(V, dtype=torch.int32)).all())
    for name, a, b in (("loss", loss, full[0]), ("lse", lse, full[1]), ("dx", dx, full[2]), ("dw", dw, full[3]),
                       ("loss_partial", lp, full[4])):
        assert same_bits(a, b), f"{name} differs from the full head"


def test_forward_only_and_argument_checks():
    import sampled_oracle as S
    from gpu_common import LOSS_TOK, O, grad_scale_dev, lib, nmce, to_dev
    T, D, V = 400, 64, 3000
    x, w, y, wt = O.make_inputs(T, D, V, seed=2, ignore_frac=0.1)
    X, W, Y, WT = to_dev(x, w, y, wt)
    gs = grad_scale_dev(WT)
    loss, lse, dx, dw, lp, cand, n = _call(X, W, Y, WT, gs, 64, 0, 464, 128, fwd=True)
    ol, olse, _, _, ocand = S.sampled_ce_f64(x, w, y, wt, float(gs.item()), 64, 0)
    assert n == ocand.size and np.abs(loss.cpu().numpy() - ol).max() <= LOSS_TOK
    with pytest.raises(nmce.NmError) as e:       # p_max below min(V, T + n_negatives) could overflow: refused
        _call(X, W, Y, WT, gs, 64, 0, 256, 128)
    assert e.value.status == 1 and "overflow" in str(e.value)
    assert lib().nm_ce_sampled_workspace_bytes(T, D, V, 463, 128, 1) == 0      # not a multiple of 8

"""Worker of the ZeRO-1 AdamH tests (one process per rank under torch.distributed.run).

  --backend gloo : CPU, oracle only. Every rank holds its own gradient of the head; the gradients are summed onto the
                   owners of each bucket's element ranges (reduce-scatter), every rank forms the partial sums of g^2,
                   p^2, a^2 over what it owns, the partials are all-reduced, owners update their elements and the
                   updated bf16 elements are all-gathered. The result must equal the single-rank oracle on the summed
                   gradient. This is the host-side contract of the sharded update, without a GPU.
  --backend nccl : GPU. The same through the library (reducer to owners + HeadAdamH), against the oracle.
"""
import argparse
import ctypes
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "marin.cpp_b200"))
import adamh_oracle as A  # noqa: E402

HY = dict(eta=0.02, b1=0.9, b2=0.98, eps=1e-20)


def inputs(V, D, world):
    rng = np.random.default_rng(42)
    w16 = torch.from_numpy((rng.standard_normal((V, D)) * 0.02).astype(np.float32)).bfloat16()
    p = w16.float().numpy()
    grads = [(rng.standard_normal((V, D)) * 1e-3).astype(np.float32) for _ in range(world)]
    mu = (rng.standard_normal((V, D)) * 1e-3).astype(np.float32)
    nu = ((rng.standard_normal((V, D)) * 1e-3) ** 2).astype(np.float32)
    return p, grads, mu, nu


def bucket_ranges(V, nb):
    tiles = (V + 127) // 128
    nb = min(nb, tiles)
    v0, v1, t0 = [], [], 0
    for b in range(nb):
        t1 = t0 + (tiles - t0) // (nb - b)
        v0.append(t0 * 128)
        v1.append(min(t1 * 128, V))
        t0 = t1
    v1[-1] = V
    return v0, v1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", required=True, choices=["gloo", "nccl"])
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    V, D, nb, t, max_norm = (700, 16, 3, 5, 0.05) if a.backend == "gloo" else (8256, 512, 5, 5, 0.5)
    p, grads, mu, nu = inputs(V, D, world)
    gsum = np.sum(np.stack(grads).astype(np.float64), axis=0).astype(np.float32) if world > 2 else \
        (grads[0] + grads[1] if world == 2 else grads[0])
    gn, clip = A.clip_state(gsum, max_norm)
    want_p, want_mu, want_nu, _ = A.adamh_f32(p, gsum, mu, nu, t, clip_gn=gn, clip=clip, max_norm=max_norm, **HY)
    v0, v1 = bucket_ranges(V, nb)
    own = A.owned_ranges(V, D, v0, v1, world, rank)

    if a.backend == "gloo":
        dist.init_process_group("gloo")
        g = torch.from_numpy(grads[rank].copy())
        dist.all_reduce(g)                                  # what the owners hold after the reduce-scatter
        g = g.numpy().reshape(-1)
        pf, muf, nuf = p.reshape(-1), mu.reshape(-1).copy(), nu.reshape(-1).copy()
        F = np.float32
        part = torch.tensor([sum(A.sumsq_f32(g[o:o + n]) for o, n in own)], dtype=torch.float64)
        dist.all_reduce(part)
        gn_r = A.norm_of(float(part.item()))
        assert not (gn_r < F(max_norm)) == clip
        sums = np.zeros(2)
        a_own = {}
        for o, n in own:                                     # pass 1 on owned elements
            gi = g[o:o + n]
            if clip:
                gi = (gi / gn_r) * F(max_norm)
            muf[o:o + n] = A.one_minus(0.9) * gi + F(0.9) * muf[o:o + n]
            nuf[o:o + n] = A.one_minus(0.98) * (gi * gi) + F(0.98) * nuf[o:o + n]
            bc1, bc2 = A.bias_correction(0.9, t), A.bias_correction(0.98, t)
            a_own[o] = muf[o:o + n] / (bc1 * (np.sqrt(nuf[o:o + n] / bc2) + F(A.decimal_of(1e-20))))
            sums += [A.sumsq_f32(pf[o:o + n]), A.sumsq_f32(a_own[o])]
        s = torch.from_numpy(sums)
        dist.all_reduce(s)
        n_, m_ = A.norm_of(float(s[0])), A.norm_of(float(s[1]))
        w_own, ww = {}, 0.0
        for o, n in own:
            w_own[o] = pf[o:o + n] - ((F(0.02) * a_own[o]) * n_) / max(m_, A.NORM_FLOOR)
            ww += A.sumsq_f32(w_own[o])
        wt = torch.tensor([ww], dtype=torch.float64)
        dist.all_reduce(wt)
        nw = A.norm_of(float(wt.item()))
        new16 = torch.zeros(V * D, dtype=torch.bfloat16)
        for o, n in own:
            pn = pf[o:o + n] + ((w_own[o] / nw) * n_ - pf[o:o + n])
            r = np.linalg.norm(pn - want_p.reshape(-1)[o:o + n]) / np.linalg.norm(want_p.reshape(-1)[o:o + n])
            assert r <= 1e-6, f"rank {rank}: owned range {o}: rel {r}"
            assert np.array_equal(muf[o:o + n], want_mu.reshape(-1)[o:o + n])
            assert np.array_equal(nuf[o:o + n], want_nu.reshape(-1)[o:o + n])
            new16[o:o + n] = torch.from_numpy(pn).bfloat16()
        gathered = new16.float()
        dist.all_reduce(gathered)                           # disjoint ranges: the sum is the all-gather
        full = torch.from_numpy(want_p.reshape(-1)).bfloat16().float()
        mism = int((gathered != full).sum())
        assert mism <= 1e-3 * V * D, f"{mism} bf16 elements differ"   # an f32 difference of 1e-7 can flip a bf16 tie
        if rank == 0:
            print(f"gloo world {world}: ZeRO-1 AdamH matches the single-rank oracle ({mism} bf16 ties)")
        dist.barrier()
        dist.destroy_process_group()
        return

    import nmce
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    lib = nmce.Lib()
    idbuf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        lib.nm_comm_unique_id(nmce.ptr(idbuf))
    idg = idbuf.to(dev)
    dist.broadcast(idg, 0)
    idbuf = idg.cpu()
    comm = ctypes.c_void_p()
    lib.nm_comm_create(nmce.ptr(idbuf), world, rank, ctypes.byref(comm))
    dw = torch.from_numpy(grads[rank]).to(dev)
    red, opt = ctypes.c_void_p(), ctypes.c_void_p()
    lib.nm_grad_reducer_create_owners(comm, nmce.ptr(dw), V, D, nb, ctypes.byref(red))
    lib.nm_head_adamh_create(V, D, red, ctypes.byref(opt))
    n_own = lib.nm_head_adamh_owned_elems(opt)
    assert n_own == V * D // world
    go, co, ln, nr = (ctypes.c_int64 * 64)(), (ctypes.c_int64 * 64)(), (ctypes.c_int64 * 64)(), ctypes.c_int(0)
    lib.nm_head_adamh_ranges(opt, 64, go, co, ln, ctypes.byref(nr))
    assert [(go[i], ln[i]) for i in range(nr.value)] == own
    idx = torch.cat([torch.arange(go[i], go[i] + ln[i]) for i in range(nr.value)])
    w16 = torch.from_numpy(p).to(dev).bfloat16()
    p_own = torch.empty(n_own, dtype=torch.float32, device=dev)
    lib.nm_head_adamh_init_master(opt, nmce.ptr(w16), nmce.ptr(p_own), None)
    assert torch.equal(p_own.cpu(), torch.from_numpy(p.reshape(-1))[idx])
    mu_own = torch.from_numpy(mu.reshape(-1))[idx].to(dev)
    nu_own = torch.from_numpy(nu.reshape(-1))[idx].to(dev)
    lib.nm_grad_reducer_reduce_all(red, None)
    lib.nm_head_adamh_step(opt, t, HY["eta"], HY["b1"], HY["b2"], HY["eps"], max_norm, 1.0, nmce.ptr(dw),
                           nmce.ptr(p_own), nmce.ptr(mu_own), nmce.ptr(nu_own), nmce.ptr(w16), None)
    torch.cuda.synchronize()
    wp = torch.from_numpy(want_p.reshape(-1))[idx]
    r = float((p_own.cpu().double() - wp.double()).norm() / wp.double().norm())
    assert r <= 1e-6, f"rank {rank}: owned p rel {r}"
    # the reduce-scatter sums the two gradients in f32 exactly as g0 + g1, so the moments are bit-equal at world 2
    if world == 2:
        assert torch.equal(mu_own.cpu(), torch.from_numpy(want_mu.reshape(-1))[idx])
        assert torch.equal(nu_own.cpu(), torch.from_numpy(want_nu.reshape(-1))[idx])
    full = torch.from_numpy(want_p).bfloat16()
    mism = int((w16.cpu() != full).sum())
    assert mism <= 1e-3 * V * D, f"rank {rank}: {mism} bf16 elements of the gathered replica differ"
    allw = [torch.empty_like(w16) for _ in range(world)]
    dist.all_gather(allw, w16)
    assert all(torch.equal(allw[0], x) for x in allw), "the replicas differ between ranks"
    # the same step with the all-gather on the communication stream: the replica is complete after wait_params and
    # bit-equal to the one gathered on the compute stream
    dw.copy_(torch.from_numpy(grads[rank]).to(dev))
    w16b = torch.from_numpy(p).to(dev).bfloat16()
    lib.nm_head_adamh_init_master(opt, nmce.ptr(w16b), nmce.ptr(p_own), None)
    mu_own.copy_(torch.from_numpy(mu.reshape(-1))[idx].to(dev))
    nu_own.copy_(torch.from_numpy(nu.reshape(-1))[idx].to(dev))
    lib.nm_grad_reducer_reduce_all(red, None)
    lib.nm_head_adamh_step_async(opt, t, HY["eta"], HY["b1"], HY["b2"], HY["eps"], max_norm, 1.0, nmce.ptr(dw),
                                 nmce.ptr(p_own), nmce.ptr(mu_own), nmce.ptr(nu_own), nmce.ptr(w16b), None)
    lib.nm_head_adamh_wait_params(opt, None)
    torch.cuda.synchronize()
    assert torch.equal(w16b, w16), f"rank {rank}: the replica gathered on the communication stream differs"
    if rank == 0:
        print(f"nccl world {world}: ZeRO-1 AdamH p rel {r:.2e}, {mism} bf16 ties")
    dist.barrier()
    lib.nm_head_adamh_destroy(opt)
    lib.nm_grad_reducer_destroy(red)
    lib.nm_comm_destroy(comm)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

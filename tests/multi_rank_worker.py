"""Worker of the multi-rank tests (launched by torch.distributed.run, one process per rank).

  --backend gloo : CPU. Every rank computes the ORACLE's dW on its row shard; the shards' sum (gloo all-reduce) must equal
                   the oracle's dW on all rows, and the global grad scale must equal 1 / sum of all weights. This
                   checks the sharding contract of the path (rows by rank, W replicated, one sum of dW) without a GPU.
  --backend nccl : GPU. Every rank runs the fused CE on its shard with the bucketed dW reducer (f32 and bf16); rank 0
                   compares the reduced dW with a single-GPU run over all rows.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", required=True, choices=["gloo", "nccl"])
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    import ce_oracle as O
    T, D, V = (96 * world, 64, 700) if a.backend == "gloo" else (1536 * world, 512, 8256)
    x, w, y, wt = O.make_inputs(T, D, V, seed=77, ignore_frac=0.1, labels="zipf")
    n = T // world
    sl = slice(rank * n, (rank + 1) * n)
    if a.backend == "gloo":
        dist.init_process_group("gloo")
        wsum = torch.tensor([float(wt[sl].sum())], dtype=torch.float64)
        dist.all_reduce(wsum)
        gs = 1.0 / float(wsum.item())
        assert abs(gs - 1.0 / float(wt.sum())) < 1e-15
        c = O.COracle()
        loss, lse, dx, dw = c.run(x[sl], w, y[sl], wt[sl], gs, z_loss=1e-4, ignore_index=-100)
        dwt = torch.from_numpy(dw)
        dist.all_reduce(dwt)
        part = torch.tensor([float((loss.astype(np.float64) * wt[sl]).sum())], dtype=torch.float64)
        dist.all_reduce(part)
        if rank == 0:
            fl, _, fdx, fdw = c.run(x, w, y, wt, gs, z_loss=1e-4, ignore_index=-100)
            r = np.linalg.norm(dwt.numpy().astype(np.float64) - fdw) / np.linalg.norm(fdw)
            assert r < 1e-5, f"sharded dW sum vs all rows: rel {r}"
            assert np.abs(fdx[sl] - dx).max() == 0, "dX rows do not depend on the other ranks"
            assert abs(float(part.item()) - float((fl.astype(np.float64) * wt).sum())) < 1e-6 * float(part.item())
            print(f"gloo world {world}: sharded oracle dW rel {r:.2e}")
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
    X = torch.from_numpy(x[sl]).to(dev).bfloat16()
    W = torch.from_numpy(w).to(dev).bfloat16()
    Y = torch.from_numpy(y[sl]).to(dev)
    WT = torch.from_numpy(wt[sl]).to(dev)
    gs = torch.tensor([1.0 / float(wt.sum())], dtype=torch.float32, device=dev)
    # bf16 wire format: every rank's dW is rounded to bf16, summed in bf16 and read back, i.e. two or three bf16
    # roundings of relative size 2^-9 / sqrt(3) each on top of the f32 result: inside the 3e-3 gradient bar
    for reduce_dtype, tol in ((0, 1e-5), (1, 3e-3)):
        dw = torch.zeros(V, D, dtype=torch.float32, device=dev)
        staging = torch.empty(V, D, dtype=torch.bfloat16, device=dev) if reduce_dtype else None
        red = ctypes.c_void_p()
        lib.nm_grad_reducer_create(comm, nmce.ptr(dw), V, D, 5, reduce_dtype, nmce.ptr(staging), ctypes.byref(red))
        dx = torch.empty_like(X)
        nmce.ce_call(lib, "B1", X, W, Y, WT, gs, dx=dx, dw=dw, chunk=512, z_loss=1e-4, ignore_index=-100, reducer=red)
        lib.nm_grad_reducer_wait(red, None)
        torch.cuda.synchronize()
        if rank == 0:
            XF = torch.from_numpy(x).to(dev).bfloat16()
            YF, WF = torch.from_numpy(y).to(dev), torch.from_numpy(wt).to(dev)
            dwf = torch.zeros(V, D, dtype=torch.float32, device=dev)
            dxf = torch.empty_like(XF)
            nmce.ce_call(lib, "B1", XF, W, YF, WF, gs, dx=dxf, dw=dwf, chunk=512, z_loss=1e-4, ignore_index=-100)
            torch.cuda.synchronize()
            r = float((dw.double() - dwf.double()).norm() / dwf.double().norm())
            assert r < tol, f"reduce dtype {reduce_dtype}: reduced dW vs single GPU rel {r}"
            assert torch.equal(dx, dxf[sl]), "dX of a shard must equal the same rows of the single-GPU run"
            print(f"nccl world {world} reduce dtype {reduce_dtype}: dW rel {r:.2e}")
        dist.barrier()
        lib.nm_grad_reducer_destroy(red)
    # ZeRO-2 for the head gradient: two microbatches per rank, an owners reducer attached to each, microbatch_done after
    # each. This rank's packed accumulator must equal its owned ranges of the all-rank, all-microbatch dW (computed by
    # every rank on all rows with plain calls; f32 sums in another order: 1e-5).
    dw = torch.zeros(V, D, dtype=torch.float32, device=dev)
    red = ctypes.c_void_p()
    lib.nm_grad_reducer_create_owners(comm, nmce.ptr(dw), V, D, 4, ctypes.byref(red))
    n_owned = int(lib.nm_grad_reducer_owned_elems(red))
    assert n_owned * world == V * D
    acc = torch.zeros(n_owned, dtype=torch.float32, device=dev)
    half = n // 2
    for m in range(2):
        rs = slice(m * half, (m + 1) * half)
        dx = torch.empty_like(X[rs])
        nmce.ce_call(lib, "B1", X[rs].contiguous(), W, Y[rs].contiguous(), WT[rs].contiguous(), gs, dx=dx, dw=dw, chunk=512,
                     z_loss=1e-4, ignore_index=-100, reducer=red)
        lib.nm_grad_reducer_microbatch_done(red, nmce.ptr(acc), None)
    torch.cuda.synchronize()
    assert not dw.any()
    XF = torch.from_numpy(x).to(dev).bfloat16()
    YF, WF = torch.from_numpy(y).to(dev), torch.from_numpy(wt).to(dev)
    dwf = torch.zeros(V, D, dtype=torch.float32, device=dev)
    nmce.ce_call(lib, "B1", XF, W, YF, WF, gs, dx=torch.empty_like(XF), dw=dwf, chunk=512, z_loss=1e-4, ignore_index=-100)
    v0 = (ctypes.c_int * 8)()
    v1 = (ctypes.c_int * 8)()
    nb = ctypes.c_int(0)
    lib.nm_grad_bucket_ranges(V, 4, v0, v1, ctypes.byref(nb))
    want = []
    for b in range(nb.value):
        nelem = (v1[b] - v0[b]) * D
        own = nelem // world
        flat = dwf[v0[b]:v1[b]].reshape(-1)
        want.append(flat[rank * own:(rank + 1) * own])
    want = torch.cat(want)
    torch.cuda.synchronize()
    r = float((acc.double() - want.double()).norm() / want.double().norm())
    assert r < 1e-5, f"ZeRO-2 owned accumulator vs all-rank dW: rel {r}"
    print(f"nccl world {world} zero2 rank {rank}: owned accumulator rel {r:.2e}")
    dist.barrier()
    lib.nm_grad_reducer_destroy(red)
    lib.nm_comm_destroy(comm)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

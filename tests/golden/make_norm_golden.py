"""Generates tests/golden/norm_golden.npz from the REFERENCE's own levanter emulation of the RMSNorm pair, imported from a
checkout of wenhaochai/marin.cpp given by --ref (this script is the only thing that reads the checkout; tests read the
.npz):

  * tests/s3/levemu.py:23-44  norm_stats, lev_norm_fwd, lev_norm_bwd: the rounding points of levanter's jaxpr written op
    by op in torch f32 with an explicit bf16 rounding after every op levanter computes in bf16;
  * the sandwich tails are composed from those three exactly as the reference's own test does
    (tests/s3/test_rmsnorm.py:158-176 sandwich_emu; that file loads the CUDA library when imported, so its twelve lines of
    composition are restated below).

    python tests/golden/make_norm_golden.py --ref /path/to/marin.cpp

Inputs follow the reference's exact-sum recipe (tests/s3/nmk.py:133-143: entries q * {-3..3} \\ {0}, gains 1 + j / 16), so
that every row sum is exact in f32 and the outputs do not depend on the order of addition; residual gradients are seeded
normal draws rounded to bf16. Runs on the CPU; sizes are kept small so the file stays a few hundred KB.
"""
import argparse
import os
import sys

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(a.ref, "tests", "s3"))
    import torch
    import levemu as E          # the reference's emulation (imports rb from its nmk.py; nothing here touches a GPU)
    from nmk import rb

    eps = float(np.float32(1e-5))   # nmk.py:299
    out = {"eps": np.float32(eps)}

    def exact_rows(T, D, gen, q=0.25):   # nmk.py:133-139 on the CPU
        v = torch.tensor((-3, -2, -1, 1, 2, 3), dtype=torch.float32)
        return (v[torch.randint(0, 6, (T, D), generator=gen)] * q).to(torch.bfloat16)

    def exact_gain(n, gen):             # nmk.py:142-143
        return (1.0 + torch.randint(-4, 5, (n,), generator=gen).float() / 16).to(torch.bfloat16)

    def bits(t):                        # bf16 tensor -> uint16 bit patterns
        return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    def bits_of_f32(t):                 # bf16-valued f32 tensor -> uint16 bit patterns
        return (t.contiguous().numpy().view(np.uint32) >> 16).astype(np.uint16)

    for name, (T, D, seed) in {"n512": (24, 512, 5), "n136": (19, 136, 6), "n2048": (9, 2048, 7)}.items():
        gen = torch.Generator().manual_seed(seed)
        x, dy = exact_rows(T, D, gen), exact_rows(T, D, gen, q=2.0 ** -8)
        g = exact_gain(D, gen)
        dres = (torch.randn(T, D, generator=gen) * 1e-2).to(torch.bfloat16)
        x32, g32, dy32 = x.float(), g.float(), dy.float()
        ms, r = E.norm_stats(x32, eps)
        oe, _ = E.lev_norm_fwd(x32, g32, r)
        dxe, dgc = E.lev_norm_bwd(x32, g32, dy32, r, ms, eps)
        out.update({f"{name}.x": bits(x), f"{name}.dy": bits(dy), f"{name}.g": bits(g), f"{name}.dres": bits(dres),
                    f"{name}.rstd": r.reshape(-1).numpy(), f"{name}.out": bits_of_f32(oe), f"{name}.dx": bits_of_f32(dxe),
                    f"{name}.dx_res": bits_of_f32(rb(dres.float() + dxe)),     # test_rmsnorm.py:64
                    f"{name}.dgc": bits_of_f32(dgc)})

    for name, (T, D, seed, post) in {"s512p": (24, 512, 8, True), "s512": (24, 512, 9, False), "s136p": (19, 136, 10, True),
                                     "s2048p": (9, 2048, 11, True)}.items():
        gen = torch.Generator().manual_seed(seed)
        b, xi = exact_rows(T, D, gen), exact_rows(T, D, gen)
        gp = exact_gain(D, gen) if post else None
        gn = exact_gain(D, gen)
        dan = exact_rows(T, D, gen, q=2.0 ** -8)
        dxo = (torch.randn(T, D, generator=gen) * 1e-2).to(torch.bfloat16)
        # test_rmsnorm.py:158-176, with the saved statistics of the forward as the backward's r
        b32, x32 = b.float(), xi.float()
        if post:
            msp, rp = E.norm_stats(b32, eps)
            y, _ = E.lev_norm_fwd(b32, gp.float(), rp)
        else:
            y = b32
        xo = rb(x32 + y)
        msn, rn = E.norm_stats(xo, eps)
        an, _ = E.lev_norm_fwd(xo, gn.float(), rn)
        dxn, dgcn = E.lev_norm_bwd(xo, gn.float(), dan.float(), rn, msn, eps)
        dxm = rb(dxo.float() + dxn)
        out.update({f"{name}.b": bits(b), f"{name}.xi": bits(xi), f"{name}.gn": bits(gn), f"{name}.dan": bits(dan),
                    f"{name}.dxo": bits(dxo), f"{name}.rn": rn.reshape(-1).numpy(), f"{name}.x_out": bits_of_f32(xo),
                    f"{name}.a_next": bits_of_f32(an), f"{name}.dx_in": bits_of_f32(dxm), f"{name}.dgcn": bits_of_f32(dgcn)})
        if post:
            dbe, dgcp = E.lev_norm_bwd(b32, gp.float(), dxm, rp, msp, eps)
            out.update({f"{name}.gp": bits(gp), f"{name}.rp": rp.reshape(-1).numpy(), f"{name}.dbranch": bits_of_f32(dbe),
                        f"{name}.dgcp": bits_of_f32(dgcp)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "norm_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()

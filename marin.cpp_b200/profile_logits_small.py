"""A small workload of the logits kernel for profilers: 4 calls of the fused CE on 4096 rows x hidden D x vocab 128256
(one chunk; about 1.7 GB on the device at D = 2048), forward-only (FWD=1: statistics, no store) or forward + backward
(FWD=0: the bf16 logits store, then the gradient pass, dW and dX). Environment: D (default 2048), FWD (default 1).

    FWD=1 ncu --set full --clock-control none -k regex:k_ce_umma -s 2 -c 1 -o prof python marin.cpp_b200/profile_logits_small.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    import torch
    import nmce
    lib = nmce.Lib()
    V, T = 128256, 4096
    D = int(os.environ.get("D", 2048))
    fwd = int(os.environ.get("FWD", 1))
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(T, D, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(V, D, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    tg = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    wt = torch.ones(T, device="cuda")
    gs = torch.full((1,), 1.0 / T, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.zeros(V, D, device="cuda")
    for _ in range(4):
        nmce.ce_call(lib, "B1", x, W, tg, wt, gs, chunk=4096, dx=None if fwd else dx, dw=None if fwd else dw,
                     forward_only=bool(fwd), check=False)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()

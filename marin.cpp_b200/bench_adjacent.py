"""Device timing of the memory-bound kernels on either side of the fused CE (RMSNorm pair, sandwich tail, doc_meta,
the in-place gradient pass) against the measured HBM copy bandwidth. One JSON line per kernel:
{"kernel", "shape", "ms", "algorithmic_bytes", "gbs", "frac_of_hbm_peak"}. Algorithmic bytes = each operand read or
written once. 5 warm-up + 20 timed launches, CUDA events on the launching stream; operands exceed L2 (126 MB).

    python marin.cpp_b200/bench_adjacent.py [--tokens 131072] [--hidden 2048]
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--hidden", type=int, default=2048)
    a = ap.parse_args()
    import torch
    import nmce
    lib = nmce.Lib()
    T, D = a.tokens, a.hidden
    peak = 6650.0
    pk = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    g = torch.Generator(device="cuda").manual_seed(1)
    bf = torch.bfloat16
    x = torch.randn(T, D, generator=g, device="cuda").to(bf)
    b = torch.randn(T, D, generator=g, device="cuda").to(bf)
    dy = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    gain = torch.ones(D, dtype=bf, device="cuda")
    y, y2, y3 = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    rstd, rstd2 = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    P = int(lib.nm_norm_partial_rows(T))
    part = torch.zeros(2 * P, D, device="cuda")
    p = nmce.ptr

    def timed(fn, n=20, w=5):
        for _ in range(w):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def report(name, ms, nbytes, shape):
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "shape": shape, "ms": round(ms, 4), "algorithmic_bytes": nbytes,
                          "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 3)}))

    TD2 = T * D * 2
    shape = f"{T} x {D} bf16"
    report("rmsnorm_fwd", timed(lambda: lib.nm_rmsnorm_fwd(1, 0, p(x), p(gain), p(y), p(rstd), T, D, 1e-5, None)),
           2 * TD2, shape)
    report("rmsnorm_bwd_add_partial",
           timed(lambda: lib.nm_rmsnorm_bwd_add_partial(1, 0, p(dy), p(x), p(gain), p(rstd), p(b), p(y2), p(part), T, D,
                                                        1e-5, None)), 4 * TD2, shape)
    report("sandwich_tail_fwd (post-norm + residual + next norm)",
           timed(lambda: lib.nm_sandwich_tail_fwd(1, 0, p(b), p(x), p(gain), p(gain), p(y), p(y2), p(rstd), p(rstd2), T,
                                                  D, 1e-5, None)), 4 * TD2, shape)
    lib.nm_sandwich_tail_fwd(1, 0, p(b), p(x), p(gain), p(gain), p(y), p(y2), p(rstd), p(rstd2), T, D, 1e-5, None)
    report("sandwich_tail_bwd (post-norm)",
           timed(lambda: lib.nm_sandwich_tail_bwd(1, 0, p(dy), p(dy), p(y), p(gain), p(rstd2), p(b), p(gain), p(rstd),
                                                  p(y3), p(y2), None, None, T, D, 1e-5, None)), 6 * TD2, shape)
    rows, S = min(16384, max(1, T // 4096)), 4096
    tok = torch.randint(0, 128000, (rows, S), generator=g, device="cuda", dtype=torch.int32)
    tg = torch.empty(rows * S, dtype=torch.int32, device="cuda")
    wt = torch.empty(rows * S, device="cuda")
    ps = torch.empty(rows * S, dtype=torch.int32, device="cuda")
    cu = torch.empty(rows * 64 + 1, dtype=torch.int32, device="cuda")
    rss = torch.empty(rows, 65, dtype=torch.int32, device="cuda")
    ns = torch.zeros(1, dtype=torch.int32, device="cuda")
    ov = torch.zeros(1, dtype=torch.int32, device="cuda")
    report("doc_meta", timed(lambda: lib.nm_doc_meta(p(tok), None, rows, S, 128001, 64, p(tg), p(wt), p(ps), p(cu), p(ns),
                                                     p(rss), p(ov), None)), 16 * rows * S, f"{rows} rows x {S}")
    V, R = 128256, 8192
    store = torch.randn(R, V, generator=g, device="cuda").to(bf)
    lse = torch.full((R,), 12.0, device="cuda")
    gsc = torch.ones(R, device="cuda")
    tgt = torch.randint(0, V, (R,), generator=g, device="cuda", dtype=torch.int32)
    report("ce_dlogits (bf16 store, in place)",
           timed(lambda: lib.nm_ce_dlogits(1, p(store), V, p(lse), p(gsc), p(tgt), R, V, None)), 4 * R * V,
           f"{R} x {V} bf16")
    del store
    # AdamH of the head, whole tensor on one GPU (N = 1) and the share of one of 8 ranks (8 owned ranges): per element
    # it reads g, p, mu, nu and writes mu, nu (pass 1: 24 B), reads p, mu, nu and writes p and its bf16 copy (pass 2:
    # 18 B), plus 4 B for the clip norm's read of g = 46 B
    import ctypes
    Dh = 2048
    for label, n_el in (("whole head, 1 rank", V * Dh), ("owned share of 1 of 8 ranks", V * Dh // 8)):
        rows = n_el // Dh
        P_ = torch.randn(rows, Dh, generator=g, device="cuda") * 0.02
        G_ = torch.randn(rows, Dh, generator=g, device="cuda") * 1e-4
        M_ = torch.zeros(rows, Dh, device="cuda")
        V_ = torch.zeros(rows, Dh, device="cuda")
        W_ = torch.empty(rows, Dh, dtype=bf, device="cuda")
        h = ctypes.c_void_p()
        lib.nm_head_adamh_create(rows, Dh, None, ctypes.byref(h))
        step = [0]

        def one():
            step[0] += 1
            lib.nm_head_adamh_step(h, step[0], 0.02, 0.9, 0.98, 1e-20, 1.0, 1.0, p(G_), p(P_), p(M_), p(V_), p(W_), None)
        report(f"head_adamh_step ({label})", timed(one), 46 * n_el, f"{rows} x {Dh} f32")
        lib.nm_head_adamh_destroy(h)
        del P_, G_, M_, V_, W_


if __name__ == "__main__":
    main()

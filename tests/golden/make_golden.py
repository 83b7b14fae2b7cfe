"""Generates tests/golden/ce_golden.npz from the REFERENCE's own Python oracles, imported from a checkout of
wenhaochai/marin.cpp given by --ref (this script is the only thing that reads the checkout; tests read the .npz):

  * tools/levref/oracle.py:101-127 cross_entropy(x, W, labels, weights, denom): float64 loss, grad_x, grad_w;
  * tests/s5/nmce.py:160-179 chunk_loss_ref(loss, w, chunk): the bit-exact emulation of the per-chunk loss tree;
  * tests/s5/test_ce.py:587-599: the exact f32 grad-scale values f32(1 / (B * 4095)) for B = 128, 256.

    python tests/golden/make_golden.py --ref /path/to/marin.cpp

Inputs are seeded numpy draws (bf16-rounded, stored as float32); sizes are kept small so the file stays a few hundred KB.
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
from ce_oracle import bf16_round  # noqa: E402  (input rounding helper only)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.ref)   # the oracle imports its siblings as tools.levref.*
    import tools.levref.oracle as levref
    sys.path.insert(0, os.path.join(a.ref, "tests", "s3"))
    sys.path.insert(0, os.path.join(a.ref, "tests", "s5"))
    import torch
    import nmce  # the reference's test helpers (module import only; nothing here touches a GPU)

    out = {}
    cases = {"a": (96, 64, 1000, 0.9, 11), "b": (70, 40, 523, 3.0, 12), "c": (33, 64, 1030, 0.45, 13)}
    for name, (T, D, V, logit_std, seed) in cases.items():
        rng = np.random.default_rng(seed)
        x = bf16_round(rng.standard_normal((T, D), dtype=np.float32))
        w = bf16_round((rng.standard_normal((V, D), dtype=np.float32) * np.float32(logit_std / D ** 0.5)))
        labels = rng.integers(0, V, size=T).astype(np.int32)
        weight = np.ones(T, np.float32)
        weight[::7] = 0.0
        weight[-1] = 0.0
        denom = float(weight.sum())
        loss, gx, gw = levref.cross_entropy(x, w, labels, weight, denom, tile=32)
        out[f"{name}_x"], out[f"{name}_w"], out[f"{name}_labels"], out[f"{name}_weight"] = x, w, labels, weight
        out[f"{name}_denom"] = np.float64(denom)
        # gradients are stored as float32 (relative storage error 6e-8, far below every bar they are checked at)
        out[f"{name}_loss"], out[f"{name}_grad_x"], out[f"{name}_grad_w"] = loss, gx.astype(np.float32), gw.astype(np.float32)
    # chunk-loss tree: random per-token losses and 0/1 weights, two chunk sizes, a ragged tail
    rng = np.random.default_rng(21)
    tl = (rng.random(5000, dtype=np.float32) * 12).astype(np.float32)
    tw = (rng.random(5000) < 0.93).astype(np.float32)
    out["tree_loss"], out["tree_weight"] = tl, tw
    for chunk in (1024, 2048, 4096):
        out[f"tree_chunk{chunk}"] = nmce.chunk_loss_ref(torch.from_numpy(tl), torch.from_numpy(tw), chunk).numpy()
    # exact grad-scale values the reference's grad_scale case checks
    for B in (128, 256):
        want = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(B * 4095), dtype=torch.float32)
        out[f"grad_scale_B{B}"] = np.float32(want.item())
    np.savez_compressed(os.path.join(HERE, "ce_golden.npz"), **out)

    # ---- doc_meta: the reference's own numpy reference, tests/s3/test_misc.py:17-36. The test module runs its
    # harness at import time, so only the source of that one function is taken from the file and executed.
    import ast
    src = open(os.path.join(a.ref, "tests", "s3", "test_misc.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "doc_meta_ref")
    ns = {"np": np}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "test_misc.py", "exec"), ns)
    doc_meta_ref = ns["doc_meta_ref"]
    EOS = 128001
    ew = {}
    rng = np.random.default_rng(0)
    rows, S, max_segs = 6, 640, 8
    tok = rng.integers(0, 128000, size=(rows, S)).astype(np.int32)
    tok[0, 0] = EOS
    tok[0, S - 1] = EOS
    tok[1, 100:103] = EOS
    tok[1, 255] = EOS
    for p_ in rng.choice(S - 1, 12, replace=False):
        tok[3, p_] = EOS
    tok[4, rng.choice(S - 1, 5, replace=False)] = EOS
    valid = np.ones(rows, bool)
    valid[5] = False
    t, w, ps, rss, cu, n, ovf = doc_meta_ref(tok, valid, EOS, max_segs)
    ew.update(dm_tok=tok, dm_valid=valid, dm_max_segs=np.int32(max_segs), dm_eos=np.int32(EOS), dm_targets=t,
              dm_weight=w, dm_pos=ps, dm_rss=rss, dm_cu=cu, dm_n=np.int32(n), dm_overflow=np.bool_(ovf))
    np.savez_compressed(os.path.join(HERE, "ew_golden.npz"), **ew)
    print("wrote", os.path.join(HERE, "ew_golden.npz"))
    print("wrote", os.path.join(HERE, "ce_golden.npz"), {k: np.asarray(v).shape for k, v in out.items()})


if __name__ == "__main__":
    main()

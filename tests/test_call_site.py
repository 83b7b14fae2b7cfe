"""The reference trainer's call site (src/model/baseline.cpp:366-373), written against this repository's C++ headers in
tests/cpp/call_site.cpp, must compile and link against the static archive (CPU check), and on a GPU give the same
numbers as the same inputs pushed through the C ABI."""
import importlib.util
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _builder():
    spec = importlib.util.spec_from_file_location("nm_build", os.path.join(ROOT, "marin.cpp_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    return b


def test_call_site_compiles_and_links():
    exe = _builder().build_call_site_example()
    assert os.path.exists(exe) and os.access(exe, os.X_OK)
    syms = subprocess.check_output(["nm", "-C", "--defined-only", exe], text=True)
    assert "nm::fused_linear_ce" in syms and "nm::ce_workspace_bytes" in syms
    assert "nm::HeadAdamH::step" in syms


def _hash_unit(i, salt):
    x = (i.astype(np.uint64) * 2654435761 + salt * 40503 + 12345) & 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 2246822519) & 0xFFFFFFFF
    x ^= x >> 13
    x = (x * 3266489917) & 0xFFFFFFFF
    x ^= x >> 16
    return ((x >> 8).astype(np.float32) * np.float32(1.0 / 8388608.0) - np.float32(1.0)).astype(np.float32)


@pytest.mark.gpu
def test_call_site_runs_and_matches_the_c_abi():
    import torch
    from gpu_common import O, nmce, run_ce
    exe = os.path.join(ROOT, "marin.cpp_b200", "call_site_example")
    if not os.path.exists(exe):
        exe = _builder().build_call_site_example()
    out = subprocess.check_output([exe], text=True, timeout=300)
    m = re.search(r"loss_sum (\S+) dw_abs (\S+) dx_abs (\S+)", out)
    assert m, out
    loss_sum, dw_abs, dx_abs = (float(v) for v in m.groups())
    T, D, V, chunk = 1500, 512, 8256, 512
    x = O.bf16_round(_hash_unit(np.arange(T * D), 1) * np.float32(1.7)).reshape(T, D)
    w = O.bf16_round(_hash_unit(np.arange(V * D), 2) * np.float32(0.035)).reshape(V, D)
    t = np.arange(T, dtype=np.uint64)
    y = ((t * 7919 + 13) % V).astype(np.int32)
    wt = np.where(t % 7 == 0, 0.0, 1.0).astype(np.float32)
    y[t % 11 == 0] = -100
    gs = np.float32(1.0) / np.float32(wt[y >= 0].sum())
    X, W = torch.from_numpy(x).cuda().bfloat16(), torch.from_numpy(w).cuda().bfloat16()
    Y, WT = torch.from_numpy(y).cuda(), torch.from_numpy(wt).cuda()
    GS = torch.tensor([gs], dtype=torch.float32, device="cuda")
    loss, lse, dx, dw, lp = run_ce(X, W, Y, WT, GS, chunk=chunk)
    assert abs(float(lp.double().sum()) * float(gs) - loss_sum) <= 1e-6 * abs(loss_sum)
    assert abs(float(dw.double().abs().sum()) - dw_abs) <= 1e-5 * dw_abs
    assert abs(float(dx.double().abs().sum()) - dx_abs) <= 1e-5 * dx_abs
    # the optimizer site: nm::HeadAdamH in the C++ program against nm_adamh_update (C ABI) on the same gradient
    m2 = re.search(r"p_abs (\S+) w16_abs (\S+)", out)
    assert m2, out
    p_abs, w16_abs = (float(v) for v in m2.groups())
    lib = nmce.Lib()
    P = W.float().contiguous()
    MU, NU = torch.zeros_like(P), torch.zeros_like(P)
    P16 = torch.empty_like(W)
    gn = float(np.sqrt(np.float32(float((dw.float() * dw.float()).double().sum()))))
    lib.nm_adamh_update(nmce.ptr(P), nmce.ptr(P16), nmce.ptr(dw), nmce.ptr(MU), nmce.ptr(NU), V, D, 1, 0.02, 0.9, 0.98,
                        1e-20, gn, int(not gn < 1.0), 1.0, None, None, None, 0, None)
    torch.cuda.synchronize()
    assert abs(float(P.double().abs().sum()) - p_abs) <= 1e-6 * p_abs
    assert abs(float(P16.double().abs().sum()) - w16_abs) <= 1e-5 * w16_abs

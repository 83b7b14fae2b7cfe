"""CPU checks of the drop-in boundary: the library loads, exports every symbol include/marincpp/*.h declares (and only
nm_* symbols), keeps the status / last-error convention, and validates arguments before touching a device. No compute
call is made here (there is no GPU and no CPU path)."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("nm_build", os.path.join(ROOT, "marin.cpp_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build()
    import nmce
    return nmce.Lib()


def declared_symbols():
    names = set()
    for h in ("capi.h", "capi_ce.h", "capi_ew.h", "capi_opt.h"):
        text = open(os.path.join(ROOT, "include", "marincpp", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(nm_[a-z0-9_]+)\s*\(", text))
    return names


def test_exports_match_headers(lib):
    out = subprocess.check_output(["nm", "-D", "--defined-only", lib.path], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if line.strip()}
    decl = declared_symbols()
    assert decl, "no declarations found"
    assert decl <= exported, f"declared but not exported: {sorted(decl - exported)}"
    assert all(s.startswith("nm_") for s in exported), f"non-nm symbols exported: {sorted(exported)[:5]}"
    assert exported <= decl, f"exported but not declared in include/: {sorted(exported - decl)}"


def test_harness_signatures_cover_headers(lib):
    import nmce
    assert set(nmce.SIGS) == declared_symbols()


def test_status_convention_without_device(lib):
    import nmce
    assert lib.nm_version().startswith(b"b200-fused-ce")
    # invalid arguments are rejected before any CUDA call, with NM_ERR_INVALID and a message
    assert lib.nm_ce_workspace_bytes(1, 1024, 2041, 1000, 256, 1) == 0
    assert b"multiple of 8" in lib.nm_last_error()
    assert lib.nm_ce_workspace_bytes(7, 1024, 512, 1000, 256, 1) == 0
    assert b"impl = 7 is not one of" in lib.nm_last_error()
    assert lib.nm_ce_workspace_bytes(1, 1024, 512, 1000, 0, 1) == 0
    nb = lib.nm_ce_workspace_bytes(1, 131072, 2048, 128256, 16384, 1)
    assert nb % 256 == 0 and nb > 16384 * 128256 * 2
    # implementation A also carries the f32-io regions, so it bounds both io layouts
    assert lib.nm_ce_workspace_bytes(0, 4096, 512, 8256, 1024, 0) > lib.nm_ce_workspace_bytes(1, 4096, 512, 8256, 1024, 0)
    args = [1, 0, 0, 1] + [None] * 10 + [0, None, None, 0, 0, 128, 512, 1000, 64, None, None]
    with pytest.raises(nmce.NmError) as e:      # io f32 with an implementation other than A
        lib.nm_fused_linear_ce(*args)
    assert e.value.status == 1 and "f32 policy of implementation A" in str(e.value)
    args[2] = 1
    with pytest.raises(nmce.NmError) as e:      # missing pointers
        lib.nm_fused_linear_ce(*args)
    assert e.value.status == 1 and "required" in str(e.value)
    args[19] = 0                                # T == 0 returns before anything else (reference ce_api.cpp:134)
    assert lib.nm_fused_linear_ce(*args) == 0
    assert lib.nm_last_error() == b""
    # set_backends returns the previous packed setting (dgrad | wgrad << 1 | sm90 << 2)
    prev = lib.nm_ce_set_backends(1, 1, -1)
    assert lib.nm_ce_set_backends(prev & 1, (prev >> 1) & 1, prev >> 2) == (3 | (prev >> 2) << 2)


def test_no_device_is_a_loud_error(lib):
    import nmce
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    assert lib.nm_device_arch() == 0 and lib.nm_last_error() != b""
    buf = (ctypes.c_float * 64)()
    with pytest.raises(nmce.NmError) as e:
        lib.nm_ce_grad_scale(ctypes.addressof(buf), 64, 1.0, ctypes.addressof(buf), None)
    assert e.value.status == 2
    # the chunk-size helper needs the SM count: 0 and a message without a device
    assert lib.nm_ce_suggest_chunk_rows(131072) == 0 and lib.nm_last_error() != b""
    # the optimizer entry points fail the same way: argument checks first, then the device
    with pytest.raises(nmce.NmError) as e:
        lib.nm_adamh_update(ctypes.addressof(buf), None, ctypes.addressof(buf), ctypes.addressof(buf),
                            ctypes.addressof(buf), 8, 8, 0, 0.02, 0.9, 0.98, 1e-20, 0.0, 0, 1.0, None, None, None, 0, None)
    assert e.value.status == 1 and "update count" in str(e.value)
    with pytest.raises(nmce.NmError) as e:
        lib.nm_adamh_update(ctypes.addressof(buf), None, ctypes.addressof(buf), ctypes.addressof(buf),
                            ctypes.addressof(buf), 8, 8, 1, 0.02, 0.9, 0.98, 1e-20, 0.0, 0, 1.0, None, None, None, 0, None)
    assert e.value.status == 2

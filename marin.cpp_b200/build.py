"""Builds marin.cpp_b200/libmarincpp_kernels.so (sm_100a only) from csrc/ with nvcc. Run as a script or call build().

    python marin.cpp_b200/build.py [--force] [--verbose]

The library is built in-tree so that it travels with the sources; only nm_* symbols are exported (csrc/capi.map).
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libmarincpp_kernels.so")
ARCHIVE = os.path.join(HERE, "libmarincpp_ce.a")
SOURCES = ["nm_core.cpp", "ce_api.cpp", "capi_ce.cpp", "comm.cpp", "ce_gemm.cu", "ce_grad_wide.cu", "ce_sampled.cu", "ce_rows.cu", "ew_rmsnorm.cu",
           "ce_static_ws.cu", "ew_sandwich.cu", "ew_norm_f32.cu", "ew_misc.cu", "opt_adamh.cu", "opt_api.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# The norm kernels restate rounding points one IEEE operation at a time: no multiply-add contraction in their units.
PER_SOURCE = {"ew_rmsnorm.cu": ["--fmad=false"], "ew_sandwich.cu": ["--fmad=false"]}
COMMON = ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-Wall",
          "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _fingerprint():
    h = hashlib.sha256()
    h.update(open(os.path.abspath(__file__), "rb").read())
    for dirpath in (CSRC, os.path.join(ROOT, "include", "marincpp"), os.path.join(ROOT, "include", "marincpp", "kernels")):
        for name in sorted(os.listdir(dirpath)):
            path = os.path.join(dirpath, name)
            if os.path.isfile(path):
                h.update(name.encode())
                h.update(open(path, "rb").read())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compiles every source for sm_100a and links the shared library. Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    stamp = os.path.join(OBJ, "fingerprint")
    fp = _fingerprint()
    if (not force and os.path.exists(LIB) and os.path.exists(ARCHIVE) and os.path.exists(stamp)
            and open(stamp).read() == fp):
        return LIB
    build_id = "b200-fused-ce-" + fp[:12]

    def compile_one(src):
        obj = os.path.join(OBJ, src + ".o")
        cmd = [NVCC] + ARCH + COMMON + ["-DNM_BUILD_ID=\"%s\"" % build_id, "-x", "cu" if src.endswith(".cu") else "c++"]
        if src.endswith(".cu"):
            cmd += ["-Xptxas", "-v"] if verbose else []
        else:
            cmd = [NVCC] + ARCH + COMMON + ["-DNM_BUILD_ID=\"%s\"" % build_id]
        cmd += PER_SOURCE.get(src, [])
        cmd += ["-c", src, "-o", obj]           # relative source name: __FILE__ in messages is the bare file name
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=CSRC)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [NVCC] + ARCH + ["-shared", "-o", LIB] + objs + [
        "-Xlinker", "--version-script=" + os.path.join(CSRC, "capi.map"), "-cudart", "static", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    # the same objects as a static archive: what a C++ host (the reference trainer) links for the nm:: API, since the
    # shared library exports only the C ABI
    if os.path.exists(ARCHIVE):
        os.remove(ARCHIVE)
    r = subprocess.run(["ar", "rcs", ARCHIVE] + objs, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("ar failed:\n%s\n%s" % (r.stdout, r.stderr))
    open(stamp, "w").write(fp)
    return LIB


def build_call_site_example(out=None):
    """Compiles tests/cpp/call_site.cpp (the reference trainer's call site against these headers) and links it with
    the static archive. Returns the executable's path."""
    build()
    out = out or os.path.join(HERE, "call_site_example")
    cmd = [NVCC] + ARCH + ["-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "call_site.cpp"), ARCHIVE, "-o", out, "-cudart", "static",
                           "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("call-site example failed to build:\n%s\n%s" % (r.stdout, r.stderr))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

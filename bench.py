"""Benchmark of the fused LM-head cross-entropy (forward + dX + dW) through the C ABI of libmarincpp_kernels.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1|c2|c3|c4] [--impl ours|reference]

One "step" is one fused-CE forward + backward over one batch of synthetic input of the named configuration (per GPU:
131072 tokens; c3 = hidden 2048 x vocab 128256, Zipf(1.1) labels, 1% ignored, z-loss 1e-4), plus, on N > 1 GPUs, the
bucketed NCCL all-reduce of dW overlapped with the last chunk's dX kernel. Rows are sharded by rank (weak scaling);
W is replicated. Rank 0 prints ONE JSON line:
  value      tokens/s of the whole job with inputs resident in HBM (CUDA events on the launching stream, max over ranks)
  e2e        the same through the same C-ABI call with HOST inputs: each step copies x, targets and weights from pinned
             host memory (double-buffered on a copy stream) and reads the per-chunk losses back
  roofline   the slowest of the three tcgen05 kernels: 2 T D V FLOP per step / its event-timed seconds per step,
             against the measured dense bf16 peak (MEASURED_PEAKS.json, sustained figure: the kernel is timed inside a
             long step); path_* are the same for the whole 6 T D V path
  cpu_baseline  the CPU oracle (oracle/ce_ref.c, OpenMP on all host cores) timed on a bounded row sample (N = 1 only)
--impl reference runs the reference itself: its fused-CE module compiled unmodified for sm_100a (oracle/_ref/, built by
oracle/Makefile where the reference's sources are present) through its own C ABI on the same configuration, on one GPU.
The reference has no CPU implementation of this path (its f32 "reference" is a GPU path too); when that library is
absent the arm falls back to timing the CPU oracle port on the host cores, a bounded row sample per step.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "marin.cpp_b200"))

CONFIGS = {
    # name: (D, V, tokens per GPU, labels, ignore fraction, z-loss, dW reduce dtype, readouts)
    "c1": dict(D=512, V=128256, T=131072, labels="uniform", ignore=0.02, z_loss=1e-4, reduce="f32", readouts=1),
    "c2": dict(D=1024, V=128256, T=131072, labels="uniform", ignore=0.02, z_loss=0.0, reduce="bf16", readouts=1),
    "c3": dict(D=2048, V=128256, T=131072, labels="zipf", ignore=0.01, z_loss=1e-4, reduce="f32", readouts=1),
    "c4": dict(D=512, V=128256, T=16384, labels="uniform", ignore=0.02, z_loss=0.0, reduce="f32", readouts=48),
}
WORKLOAD = {
    "c1": "fused CE fwd+bwd, 131072 tok/GPU x hidden 512 x vocab 128256 (Qwen3-130m head), bf16, uniform labels 2% ignored, z-loss 1e-4",
    "c2": "fused CE fwd+bwd, 131072 tok/GPU x hidden 1024 x vocab 128256 (Qwen3-520m head), bf16, uniform labels 2% ignored, bf16 dW all-reduce",
    "c3": "fused CE fwd+bwd, 131072 tok/GPU x hidden 2048 x vocab 128256 (Qwen3-1.2B head), bf16, Zipf(1.1) labels 1% ignored, z-loss 1e-4",
    "c4": "48 readouts x 16384 tok/GPU x hidden 512 x vocab 128256 (pls shared head), bf16, one dW all-reduce per step",
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_inputs(torch, cfg, rank, device, layer=0):
    """Seeded synthetic inputs of the configuration on the device: x rows ~ N(0,1) RMS-normalised, W ~ N(0, 0.02^2),
    bf16; labels uniform or Zipf(1.1) with a fraction set to -100; weight = 1[label != -100]. W and the labels do not
    depend on `layer`; x does (independent readout states)."""
    T, D, V = cfg["T"], cfg["D"], cfg["V"]
    gw = torch.Generator(device=device).manual_seed(0xC0DE)
    W = (torch.randn(V, D, generator=gw, device=device) * 0.02).to(torch.bfloat16)
    gx = torch.Generator(device=device).manual_seed(1000 + 97 * rank + layer)
    X = torch.randn(T, D, generator=gx, device=device)
    X = (X / X.pow(2).mean(dim=1, keepdim=True).sqrt()).to(torch.bfloat16)
    gy = torch.Generator(device=device).manual_seed(5000 + rank)
    if cfg["labels"] == "zipf":
        # inverse-CDF Zipf(1.1) over ranks 1..V from seeded uniforms; rank 1 is id 0
        pk = 1.0 / torch.arange(1, V + 1, dtype=torch.float64, device=device) ** 1.1
        cdf = torch.cumsum(pk, 0)
        cdf = cdf / cdf[-1]
        u = torch.rand(T, generator=gy, device=device, dtype=torch.float64)
        Y = torch.searchsorted(cdf, u, right=True).clamp_(max=V - 1).to(torch.int32)
    else:
        Y = torch.randint(0, V, (T,), generator=gy, device=device, dtype=torch.int32)
    Y[torch.rand(T, generator=gy, device=device) < cfg["ignore"]] = -100
    WT = (Y != -100).float()
    return X, W, Y, WT


def cpu_sample(cfg, seconds=12.0, rows0=32):
    """Times the CPU oracle on the first rows of rank 0's batch; returns (tokens/s, rows, threads, seconds)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ce_oracle as O
    c = O.COracle()
    D, V = cfg["D"], cfg["V"]
    x, w, y, wt = O.make_inputs(1024, D, V, seed=0xC3, ignore_frac=cfg["ignore"], labels=cfg["labels"])
    dw = None

    def run(n):
        nonlocal dw
        t = time.perf_counter()
        _, _, _, dw = c.run(x[:n], w, y[:n], wt[:n], 1.0 / max(1.0, float(wt[:n].sum())), z_loss=cfg["z_loss"],
                            ignore_index=-100, dw_out=dw)
        return time.perf_counter() - t
    t0 = run(rows0)
    n = int(max(rows0, min(1024, rows0 * seconds / max(t0, 1e-3))))
    n -= n % 4
    t1 = run(n)
    return n / t1, n, c.threads(), t1


REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_ce.so")

# DRAM bytes (read + write) per launch of the dominant tensor-core kernel, from hardware counters
# (dram__bytes_read.sum + dram__bytes_write.sum). Hidden 2048 (128 x 256-tile kernels, unchanged since): one capture of
# full chunks, {chunk rows: {kernel: bytes}}. Other shapes: the ratio of measured to algorithmic bytes seen on a small
# case (one chunk of 4096 rows), applied to the algorithmic bytes of a full launch.
FULL_SIZE_TRAFFIC = {(2048, 128256, 18944): {"logits": 7.60e9, "dw": 11.34e9, "dx": 9.26e9},
                     (2048, 128256, 16384): {"logits": 6.40e9, "dw": 10.07e9, "dx": 8.04e9}}
SMALL_CASE_RATIO = {(1024, 128256): {"logits": 0.97, "dw": 0.98, "dx": 1.07},
                    (512, 128256): {"logits": 0.96, "dw": 0.98, "dx": 1.00}}


def dram_traffic_per_launch(kernel, D, V, chunk, grad_path):
    full = FULL_SIZE_TRAFFIC.get((D, V, chunk), {}).get(kernel)
    if full is not None and grad_path in (-1, 0):
        return full
    ratio = SMALL_CASE_RATIO.get((D, V), {}).get(kernel)
    if ratio is None or grad_path not in (-1, 2):
        return None
    store = 2.0 * chunk * V
    algorithmic = {"logits": 2.0 * chunk * D + 2.0 * V * D + store + 8.0 * chunk * ((V + 255) // 256),
                   "dw": store + 2.0 * chunk * D + 8.0 * V * D,
                   "dx": store + 2.0 * V * D + 2.0 * chunk * D}[kernel]
    return ratio * algorithmic


def reference_arm_gpu(args, cfg):
    """The reference's own fused-CE module (compiled unmodified for sm_100a by oracle/Makefile into oracle/_ref/),
    driven through its C ABI on the full configuration: implementation B1, bf16 store, default backends (cuBLASLt for
    the plain-dz GEMMs, its portable mma.sync logits kernel), i.e. what its trainer would run on this GPU."""
    import torch
    import nmce
    dll = ctypes.CDLL(REF_LIB)
    for n in ("nm_ce_workspace_bytes", "nm_fused_linear_ce", "nm_last_error"):
        f = getattr(dll, n)
        f.restype, f.argtypes = nmce.SIGS[n]
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    T, D, V = cfg["T"], cfg["D"], cfg["V"]
    R = cfg["readouts"]
    X, W, Y, WT = make_inputs(torch, cfg, 0, dev)
    gs = (1.0 / WT.sum()).float().reshape(1) / R
    dx = torch.empty_like(X)
    dw = torch.zeros(V, D, dtype=torch.float32, device=dev)
    loss = torch.empty(T, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    # chunk sizes: the one passed; else both the value the reference's own callers use (16384, tests/s5/bench_ce.py)
    # and the one the other arm of this bench runs by default (128 x SM count): the faster of the two is reported
    chunks = [min(args.chunk, T)] if args.chunk else sorted({min(16384, T), min(128 * sms, T)})

    def run(chunk, warmup, steps):
        lp = torch.zeros((T + chunk - 1) // chunk, dtype=torch.float32, device=dev)
        ws = torch.empty(dll.nm_ce_workspace_bytes(1, T, D, V, chunk, 1), dtype=torch.uint8, device=dev)

        def step():
            dw.zero_()
            for _ in range(R):
                r = dll.nm_fused_linear_ce(1, 0, 1, 1, nmce.ptr(X), nmce.ptr(W), nmce.ptr(Y), nmce.ptr(WT),
                                           nmce.ptr(gs), None, nmce.ptr(loss), nmce.ptr(lse), nmce.ptr(lp), nmce.ptr(dx),
                                           0, nmce.ptr(dw), None, 0, 0, T, D, V, chunk, nmce.ptr(ws), sp)
                if r != 0:
                    raise RuntimeError("reference nm_fused_linear_ce: " + dll.nm_last_error().decode())
        for _ in range(max(1, warmup)):
            step()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        del ws
        return e0.elapsed_time(e1)

    tried = {}
    if len(chunks) > 1:                       # a short look at each, then the full measurement on the faster one
        for c in chunks:
            tried[str(c)] = run(c, 2, 3) / 3
        chunk = int(min(tried, key=tried.get))
    else:
        chunk = chunks[0]
    sampler = ClockSampler(0)
    sampler.start()
    ms = run(chunk, args.warmup, args.steps)
    clocks = sampler.stop()
    val = R * T * args.steps / (ms * 1e-3)
    sample = ("GPU run, not CPU: the reference has no CPU implementation of this path; this is its own CE module "
              "(B1, bf16 store, cuBLASLt + mma.sync) built unmodified for sm_100a, full configuration, one GPU")
    print(json.dumps({
        "impl": "reference", "metric": "fused_ce_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD[args.config], "tokens_per_gpu": R * T, "hidden": D, "vocab": V,
                   "chunk_rows": chunk, "chunk_rows_tried_ms_per_step": tried or None,
                   "z_loss": "unsupported by the reference API (its fused CE has no z-loss term): run without it",
                   "note": "rank 0 only: the reference's CE module on one GPU (its trainer's multi-GPU loop is not "
                           "part of this path); per-GPU throughput, to be compared with the other arm's value / n_gpus",
                   "path_tflops": 6.0 * R * T * D * V / (ms / args.steps * 1e-3) / 1e12},
        "clocks": clocks,
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": 0, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def reference_arm(args, cfg, rank, world):
    """The reference arm. When the reference's own CE module has been built (oracle/_ref/libref_ce.so) and a GPU is
    present, that is what runs (see reference_arm_gpu). Otherwise: the reference has no CPU implementation of this
    path, so the arm times the CPU oracle port (oracle/ce_ref.c) on the host cores, a bounded row sample per step."""
    if rank != 0:
        return
    if os.path.exists(REF_LIB):
        try:
            import torch
            if torch.cuda.is_available():
                reference_arm_gpu(args, cfg)
                return
        except (OSError, RuntimeError) as e:   # fall through to the CPU port, saying why
            sys.stderr.write(f"reference library unusable ({e}); timing the CPU oracle port instead\n")
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ce_oracle as O
    c = O.COracle()
    D, V = cfg["D"], cfg["V"]
    rows = 64
    x, w, y, wt = O.make_inputs(rows, D, V, seed=0xC3, ignore_frac=cfg["ignore"], labels=cfg["labels"])
    gs = 1.0 / max(1.0, float(wt.sum()))
    dw = None
    for _ in range(args.warmup):
        _, _, _, dw = c.run(x, w, y, wt, gs, z_loss=cfg["z_loss"], ignore_index=-100, dw_out=dw)
    t = time.perf_counter()
    for _ in range(args.steps):
        _, _, _, dw = c.run(x, w, y, wt, gs, z_loss=cfg["z_loss"], ignore_index=-100, dw_out=dw)
    dt = time.perf_counter() - t
    val = rows * args.steps / dt
    sample = f"{rows} rows of the {args.config} batch per step (cost is linear in rows), full vocabulary"
    print(json.dumps({
        "impl": "reference", "metric": "fused_ce_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD[args.config], "note": "CPU oracle port on the host cores; the reference ships "
                   "no CPU implementation of this path"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": c.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def measure(args, cfg, name, env, steps, warmup, with_e2e):
    """One configuration on this rank's GPU: device-resident timing (+ the host-input leg when asked). Returns a dict of
    raw numbers; every rank calls it, the collectives inside need all of them."""
    torch, nmce, lib, dist, rank, world, dev = (env[k] for k in ("torch", "nmce", "lib", "dist", "rank", "world", "dev"))
    T, D, V, L = cfg["T"], cfg["D"], cfg["V"], cfg["z_loss"]
    R = cfg["readouts"]
    chunk = min(args.chunk or int(lib.nm_ce_suggest_chunk_rows(T)), T)
    n_chunks = (T + chunk - 1) // chunk

    X, W, Y, WT = make_inputs(torch, cfg, rank, dev)
    Xs = [X] + [make_inputs(torch, cfg, rank, dev, layer=l)[0] for l in range(1, R)]
    wsum = WT.sum().double().reshape(1)
    if dist:
        dist.all_reduce(wsum)
    gs = (1.0 / wsum).float().to(dev)                      # global mean over non-ignored tokens (and readouts below)
    if R > 1:
        gs = gs / R
    dx = torch.empty_like(X)
    dw = torch.zeros(V, D, dtype=torch.float32, device=dev)
    loss = torch.empty(T, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    lp = torch.zeros(R, n_chunks, dtype=torch.float32, device=dev)
    ws = torch.empty(lib.nm_ce_workspace_bytes(1, T, D, V, chunk, 1), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    sp = ctypes.c_void_p(stream.cuda_stream)

    comm, reducer, staging = env.get("comm"), None, None
    if world > 1:
        if cfg["reduce"] == "bf16":
            staging = torch.empty(V, D, dtype=torch.bfloat16, device=dev)
        reducer = ctypes.c_void_p()
        if args.zero1:
            lib.nm_grad_reducer_create_owners(comm, nmce.ptr(dw), V, D, args.buckets, ctypes.byref(reducer))
        else:
            lib.nm_grad_reducer_create(comm, nmce.ptr(dw), V, D, args.buckets, 1 if cfg["reduce"] == "bf16" else 0,
                                       nmce.ptr(staging), ctypes.byref(reducer))
    head_opt = None
    if args.zero1:
        head_opt = ctypes.c_void_p()
        lib.nm_head_adamh_create(V, D, reducer, ctypes.byref(head_opt))
        n_own = int(lib.nm_head_adamh_owned_elems(head_opt))
        p_own = torch.empty(n_own, dtype=torch.float32, device=dev)
        mu_own = torch.zeros(n_own, dtype=torch.float32, device=dev)
        nu_own = torch.zeros(n_own, dtype=torch.float32, device=dev)
        lib.nm_head_adamh_init_master(head_opt, nmce.ptr(W), nmce.ptr(p_own), sp)
        opt_t = [0]

    def ce(x_in, y_in, wt_in, r, last):
        lib.nm_fused_linear_ce_ex(1, 0, 1, 1, nmce.ptr(x_in), nmce.ptr(W), nmce.ptr(y_in), nmce.ptr(wt_in),
                                  nmce.ptr(gs), None, nmce.ptr(loss), nmce.ptr(lse), nmce.ptr(lp[r]), nmce.ptr(dx), 0,
                                  nmce.ptr(dw), None, 0, int(args.forward_only), T, D, V, chunk, nmce.ptr(ws), sp, float(L),
                                  -100, reducer if (last and not args.forward_only) else None)

    if R > 1:   # pls: every layer's readout state goes through the readout entry point (norm + CE + norm backward)
        gain = torch.ones(D, dtype=torch.bfloat16, device=dev)
        norm_out = torch.empty_like(X)
        norm_rstd = torch.empty(T, dtype=torch.float32, device=dev)
        d_state = torch.zeros_like(X)
        dgain_part = torch.zeros(int(lib.nm_norm_partial_rows(T)), D, dtype=torch.float32, device=dev)

    def readout(x_in, y_in, wt_in, r):
        lib.nm_ce_readout(1, 0, 1, nmce.ptr(x_in), nmce.ptr(gain), nmce.ptr(norm_rstd), nmce.ptr(norm_out),
                          nmce.ptr(W), nmce.ptr(dw), nmce.ptr(dgain_part), nmce.ptr(gs), nmce.ptr(d_state), D,
                          nmce.ptr(y_in), nmce.ptr(wt_in), nmce.ptr(loss), nmce.ptr(lse), nmce.ptr(lp[r]), 0, T, D, V,
                          chunk, 1e-5, nmce.ptr(ws), sp)

    comm_events = None       # pairs of events around the wait for the dW all-reduce (its exposed, non-overlapped part)
    other_launches = [0]     # launches per step outside the six timed kernel classes (norms, casts, optimizer)
    if R > 1:
        other_launches[0] += R * 2                         # the readout's RMSNorm forward and backward
    if reducer and cfg["reduce"] == "bf16":
        other_launches[0] += 2 * args.buckets              # casts around the bf16 all-reduce
    if args.zero1:
        other_launches[0] += 5                             # AdamH: clip norm + its partial sum, moments + sums, apply

    def step(inputs=None):
        """zero dW, every readout's fused CE (dW accumulates), the dW all-reduce overlapped with the last dX (one
        readout) or issued once after the last readout (pls)."""
        dw.zero_()
        for r in range(R):
            x_in, y_in, wt_in = inputs if inputs is not None else (Xs[r], Y, WT)
            if R > 1:
                readout(x_in, y_in, wt_in, r)
            else:
                ce(x_in, y_in, wt_in, r, last=True)
        if reducer:
            if R > 1:
                lib.nm_grad_reducer_reduce_all(reducer, sp)
            if comm_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                comm_events.append(ev)
            lib.nm_grad_reducer_wait(reducer, sp)
            if comm_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                comm_events.append(ev)
        if head_opt:
            opt_t[0] += 1     # a tiny learning rate: the master copy moves every step, the synthetic loss stays where it is
            lib.nm_head_adamh_step(head_opt, opt_t[0], 1e-6, 0.9, 0.98, 1e-20, 1.0, 1.0, nmce.ptr(dw), nmce.ptr(p_own),
                                   nmce.ptr(mu_own), nmce.ptr(nu_own), nmce.ptr(W), sp)

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def check_status():
        st = ctypes.c_uint32(0)
        lib.nm_ce_device_status(nmce.ptr(ws), sp, ctypes.byref(st))

    # ---------------------------------------------------------------- device-resident timing (value)
    for _ in range(warmup):
        step()
    check_status()
    lib.nm_ce_profile_enable(R * (n_chunks * 6 + args.buckets) * steps + 64)
    sampler = ClockSampler(env["local_rank"])
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    comm_events = [] if reducer else None
    e0.record(stream)
    step_marks = []
    for _ in range(steps):
        step()
        m = torch.cuda.Event(enable_timing=True)
        m.record(stream)
        step_marks.append(m)
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    # per-step durations on this rank (the headline stays the total over the K steps, max over ranks)
    per_step = [a.elapsed_time(b) for a, b in zip([e0] + step_marks[:-1], step_marks)]
    exposed_comm_ms = None
    if comm_events:
        exposed_comm_ms = sum(comm_events[i].elapsed_time(comm_events[i + 1])
                              for i in range(0, len(comm_events), 2)) / steps
    comm_events = None
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    exposed_by_rank = clocks_by_rank = None
    if dist:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        # every rank's wait for the all-reduce beside its clock: the ranks' GPUs run at different power-capped clocks,
        # and the faster ones wait here for the slowest one's last bucket (the smallest wait is what the collective
        # itself exposes)
        ex = torch.tensor([exposed_comm_ms or 0.0, float(clocks.get("sm_mhz") or 0.0)], dtype=torch.float64, device=dev)
        allex = [torch.zeros_like(ex) for _ in range(world)]
        dist.all_gather(allex, ex)
        exposed_by_rank = [round(float(t[0].item()), 3) for t in allex]
        clocks_by_rank = [float(t[1].item()) for t in allex]
    ms_total = float(ms.item())
    prof_ms = (ctypes.c_double * 6)()
    prof_n = (ctypes.c_int * 6)()
    lib.nm_ce_profile_read(prof_ms, prof_n)
    lib.nm_ce_profile_enable(0)
    check_status()
    lsum = lp.double().sum().reshape(1)
    if dist:
        dist.all_reduce(lsum)
    loss_value = float((lsum * gs.double()).item())         # global weighted mean loss of the last step

    # ---------------------------------------------------------------- host-input timing (e2e)
    e2e = None
    if with_e2e:
        hx = [torch.empty(T, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        hy = [torch.empty(T, dtype=torch.int32).pin_memory() for _ in range(2)]
        hw = [torch.empty(T, dtype=torch.float32).pin_memory() for _ in range(2)]
        for b in range(2):
            hx[b].copy_(X)
            hy[b].copy_(Y)
            hw[b].copy_(WT)
        dxin = [torch.empty_like(X) for _ in range(2)]
        dyin = [torch.empty_like(Y) for _ in range(2)]
        dwin = [torch.empty_like(WT) for _ in range(2)]
        hlp = torch.empty(R, n_chunks, dtype=torch.float32).pin_memory()
        copy_stream = torch.cuda.Stream(dev)
        ready = [torch.cuda.Event() for _ in range(2)]
        freed = [torch.cuda.Event() for _ in range(2)]

        def upload(b):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(freed[b])
                dxin[b].copy_(hx[b], non_blocking=True)
                dyin[b].copy_(hy[b], non_blocking=True)
                dwin[b].copy_(hw[b], non_blocking=True)
                ready[b].record(copy_stream)

        def e2e_steps(k):
            for b in range(2):
                freed[b].record(stream)
            upload(0)
            for i in range(k):
                b = i & 1
                if i + 1 < k:
                    upload(b ^ 1)                       # next step's inputs travel while this step computes
                stream.wait_event(ready[b])
                step((dxin[b], dyin[b], dwin[b]))
                freed[b].record(stream)
                hlp.copy_(lp, non_blocking=True)        # the step's result: per-chunk weighted losses
            stream.synchronize()

        e2e_steps(warmup)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        e2e_steps(steps)
        f1.record(stream)
        barrier()
        ms2 = torch.tensor([f0.elapsed_time(f1)], dtype=torch.float64, device=dev)
        if dist:
            dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        check_status()
        h2d = T * D * 2 + T * 4 + T * 4                  # one upload of x, targets, weights per step
        e2e = {"value": world * R * T * steps / (float(ms2.item()) * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": R * n_chunks * 4,
               "ms_per_step": float(ms2.item()) / steps}

    if head_opt:
        lib.nm_head_adamh_destroy(head_opt)
    if reducer:
        lib.nm_grad_reducer_destroy(reducer)
    pk = peaks()
    names = ["logits", "finalize", "dlogits", "dw", "dx", "chunk_loss"]
    per_class = {names[i]: {"ms_per_step": prof_ms[i] / steps, "launches_per_step": prof_n[i] / steps}
                 for i in range(6)}
    ms_step = ms_total / steps
    path_tflops = 6.0 * R * T * D * V / (ms_step * 1e-3) / 1e12
    return dict(name=name, T=T, D=D, V=V, R=R, chunk=chunk, n_chunks=n_chunks, ms_total=ms_total, ms_step=ms_step,
                per_step=per_step, clocks=clocks, clocks_by_rank=clocks_by_rank, exposed_comm_ms=exposed_comm_ms,
                exposed_by_rank=exposed_by_rank, prof_ms=list(prof_ms), prof_n=list(prof_n), per_class=per_class,
                loss=loss_value, e2e=e2e, launches=int(sum(prof_n)) + other_launches[0] * steps,
                path_tflops=path_tflops, path_frac=path_tflops / pk["sustained"],
                path_frac_of_burst=path_tflops / pk["burst"], tokens_per_s=world * R * T * steps / (ms_total * 1e-3))


def adjacent_kernels(env, tokens=65536, hidden=2048):
    """The memory-bound kernels on either side of the fused CE (RMSNorm pair, sandwich tail, the in-place gradient
    pass, the head's AdamH), each timed alone over operands larger than L2: GB/s of algorithmic bytes (every operand read
    or written once) and the fraction of the measured HBM copy rate. 3 warm-up + 10 timed launches, CUDA events."""
    torch, nmce, lib = env["torch"], env["nmce"], env["lib"]
    peak = peaks()["hbm"]
    T, D = tokens, hidden
    g = torch.Generator(device="cuda").manual_seed(1)
    bf = torch.bfloat16
    x = torch.randn(T, D, generator=g, device="cuda").to(bf)
    b = torch.randn(T, D, generator=g, device="cuda").to(bf)
    dy = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    dy2 = (torch.randn(T, D, generator=g, device="cuda") * 1e-2).to(bf)
    gain = torch.ones(D, dtype=bf, device="cuda")
    y, y2, y3 = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    rstd, rstd2 = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    P = int(lib.nm_norm_partial_rows(T))
    part = torch.zeros(2 * P, D, device="cuda")
    p = nmce.ptr
    out = {}

    def timed(name, nbytes, fn, n=10, w=3):
        for _ in range(w):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 3)}

    TD2 = T * D * 2
    timed("rmsnorm_fwd", 2 * TD2, lambda: lib.nm_rmsnorm_fwd(1, 0, p(x), p(gain), p(y), p(rstd), T, D, 1e-5, None))
    timed("rmsnorm_bwd_add_partial", 4 * TD2,
          lambda: lib.nm_rmsnorm_bwd_add_partial(1, 0, p(dy), p(x), p(gain), p(rstd), p(b), p(y2), p(part), T, D, 1e-5,
                                                 None))
    timed("sandwich_tail_fwd", 4 * TD2,
          lambda: lib.nm_sandwich_tail_fwd(1, 0, p(b), p(x), p(gain), p(gain), p(y), p(y2), p(rstd), p(rstd2), T, D,
                                           1e-5, None))
    timed("sandwich_tail_bwd", 6 * TD2,
          lambda: lib.nm_sandwich_tail_bwd_partial(1, 0, p(dy), p(dy2), p(y), p(gain), p(rstd2), p(b), p(gain), p(rstd),
                                                   p(y3), p(y2), p(part), p(part[P:]), T, D, 1e-5, None))
    V, Rr = 128256, 4096
    store = torch.randn(Rr, V, generator=g, device="cuda").to(bf)
    lse = torch.full((Rr,), 12.0, device="cuda")
    gsc = torch.ones(Rr, device="cuda")
    tgt = torch.randint(0, V, (Rr,), generator=g, device="cuda", dtype=torch.int32)
    timed("ce_dlogits_inplace", 4 * Rr * V, lambda: lib.nm_ce_dlogits(1, p(store), V, p(lse), p(gsc), p(tgt), Rr, V, None))
    del store
    rows = V // 4
    P_ = torch.randn(rows, D, generator=g, device="cuda") * 0.02
    G_ = torch.randn(rows, D, generator=g, device="cuda") * 1e-4
    M_, V_ = torch.zeros(rows, D, device="cuda"), torch.zeros(rows, D, device="cuda")
    W_ = torch.empty(rows, D, dtype=bf, device="cuda")
    h = ctypes.c_void_p()
    lib.nm_head_adamh_create(rows, D, None, ctypes.byref(h))
    t_opt = [0]

    def one():
        t_opt[0] += 1
        lib.nm_head_adamh_step(h, t_opt[0], 0.02, 0.9, 0.98, 1e-20, 1.0, 1.0, p(G_), p(P_), p(M_), p(V_), p(W_), None)
    timed("head_adamh_step", 46 * rows * D, one)     # 24 + 18 bytes per element in two passes + 4 for the clip norm
    lib.nm_head_adamh_destroy(h)
    out["shape"] = f"{T} x {D} bf16 (dlogits {Rr} x {V}; AdamH {rows} x {D} f32)"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunk", type=int, default=0, help="chunk rows; 0 = nm_ce_suggest_chunk_rows (128 x SM count)")
    ap.add_argument("--buckets", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (small cases for profiling)")
    ap.add_argument("--cta-pair", default="", help="three digits (logits, dX, dW): 1 = a CTA pair per tile, 0 = one CTA, e.g. 011; default: chosen per launch")
    ap.add_argument("--grad-path", type=int, default=-1,
                    help="how dX / dW get the normalised gradient: 0 in-place pass + 128x256 tiles, 1 pass + 256x512 pair "
                         "tiles, 2 formed inside the pair-tile kernels (no pass); -1: chosen per call")
    ap.add_argument("--tail-order", type=int, default=0,
                    help="last chunk with a dW reducer: 0 dW buckets first and dX beside their reductions; 1 dX first on "
                         "all SMs, then dW buckets beside the reductions")
    ap.add_argument("--zero1", action="store_true",
                    help="reduce dW to its owners (reduce-scatter), AdamH on owned elements and all-gather of the bf16 "
                         "head inside every step, instead of the dW all-reduce (the optimizer then is in the timing)")
    ap.add_argument("--forward-only", action="store_true",
                    help="statistics and loss only (the evaluation path; also the small case of the logits kernel without its store)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input leg")
    ap.add_argument("--adjacent-only", action="store_true",
                    help="time only the memory-bound neighbours (RMSNorm pair, sandwich tail, in-place pass, AdamH) and "
                         "print their JSON: a small case of those kernels for profiling")
    ap.add_argument("--no-others", action="store_true",
                    help="skip the short runs of the other configurations and of the neighbouring memory-bound kernels")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.tokens > 0:
        cfg["T"] = args.tokens
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.warmup < 3:
        args.warmup = 3 if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        reference_arm(args, cfg, rank, world)
        return

    # stdout carries the one JSON line: whatever NCCL is asked to log goes to stderr unless a file was named
    if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
        os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
    import torch
    import nmce
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = nmce.Lib()
    if args.cta_pair:
        lib.nm_ce_set_cta_pair(*[int(ch) for ch in args.cta_pair])
    lib.nm_ce_set_grad_path(args.grad_path)
    lib.nm_ce_set_tail_order(args.tail_order)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    env = dict(torch=torch, nmce=nmce, lib=lib, dist=dist, rank=rank, world=world, dev=dev, local_rank=local_rank)
    if args.adjacent_only:
        print(json.dumps({"adjacent": adjacent_kernels(env, args.tokens or 65536, cfg["D"])}))
        return
    if world > 1:
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            lib.nm_comm_unique_id(nmce.ptr(idbuf))
        idg = idbuf.to(dev)
        dist.broadcast(idg, 0)
        idbuf = idg.cpu()
        comm = ctypes.c_void_p()
        lib.nm_comm_create(nmce.ptr(idbuf), world, rank, ctypes.byref(comm))
        env["comm"] = comm

    m = measure(args, cfg, args.config, env, args.steps, args.warmup, not args.no_e2e)

    # the other configurations, three timed steps each, and the memory-bound neighbours: one GPU, default run only
    others = adjacent = None
    if world == 1 and not args.no_others and args.tokens == 0:
        others = {}
        for name in sorted(CONFIGS):
            if name == args.config:
                continue
            o = measure(args, dict(CONFIGS[name]), name, env, 3, 3, False)
            others[name] = {"ms_per_step": o["ms_step"], "tokens_per_s": o["tokens_per_s"], "chunk_rows": o["chunk"],
                            "path_tflops": o["path_tflops"], "path_frac": o["path_frac"],
                            "path_frac_of_burst": o["path_frac_of_burst"], "sm_mhz": o["clocks"].get("sm_mhz"),
                            "per_kernel_class": o["per_class"], "loss": o["loss"]}
            del o
            torch.cuda.empty_cache()
        adjacent = adjacent_kernels(env)

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, n, threads, secs = cpu_sample(cfg)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"first {n} rows of the batch, full vocabulary, {secs:.1f} s (cost is linear in rows)"}

    if world > 1:
        lib.nm_comm_destroy(env["comm"])
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    pk = peaks()
    T, D, V, R, chunk = m["T"], m["D"], m["V"], m["R"], m["chunk"]
    names = ["logits", "finalize", "dlogits", "dw", "dx", "chunk_loss"]
    gemm = {k: m["per_class"][k]["ms_per_step"] for k in ("logits", "dw", "dx")}
    dom = max(gemm, key=gemm.get)
    di = names.index(dom)
    dom_launch_ms = m["prof_ms"][di] / max(1, m["prof_n"][di])
    dom_flop_launch = 2.0 * R * T * D * V * args.steps / max(1, m["prof_n"][di])
    achieved = dom_flop_launch / (dom_launch_ms * 1e-3) / 1e12
    out = {
        "metric": "fused_ce_fwd_bwd_tokens_per_s", "value": m["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms_step"],
        "ms_per_step_median_rank0": sorted(m["per_step"])[len(m["per_step"]) // 2],
        "ms_per_step_min_rank0": min(m["per_step"]),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD[args.config] + (f" [tokens overridden to {T}]" if args.tokens > 0 else ""),
                   "tokens_per_gpu": R * T, "hidden": D, "vocab": V,
                   "chunk_rows": chunk, "readouts": R, "grad_path": args.grad_path, "tail_order": args.tail_order, "forward_only": args.forward_only,
                   "parallelism": f"dp{world} (rows sharded, W replicated)",
                   "dw_allreduce": ((f"f32 reduce-scatter to owners, {args.buckets} buckets, overlapped with the last dX"
                                     if args.zero1 else
                                     f"{cfg['reduce']}, {args.buckets} buckets, overlapped with the last dX")
                                    if world > 1 else "none (1 GPU)"),
                   "optimizer_in_step": ("AdamH of the head on owned elements + bf16 all-gather (ZeRO-1)"
                                         if args.zero1 else None),
                   "exposed_allreduce_ms_per_step_rank0": m["exposed_comm_ms"],
                   "allreduce_wait_ms_per_step_by_rank": m["exposed_by_rank"],
                   "sm_mhz_median_by_rank": m["clocks_by_rank"],
                   "l2": "inputs (x, W, logits store: > 5 GB per step) exceed the 126 MB L2; no flush needed",
                   "loss": m["loss"]},
        "clocks": m["clocks"],
        "e2e": m["e2e"],
        "gpu_launches": m["launches"],
        "roofline": {"bound": "tensor", "kernel": f"k_ce_{dom}", "achieved": achieved, "peak": pk["sustained"],
                     "unit": "TFLOP/s", "frac": achieved / pk["sustained"],
                     "traffic": dram_traffic_per_launch(dom, D, V, chunk, args.grad_path),
                     "peak_source": f"{pk['source']} (sustained; burst {pk['burst']})",
                     "frac_of_burst": achieved / pk["burst"], "launch_ms": dom_launch_ms,
                     "path_tflops": m["path_tflops"], "path_frac": m["path_frac"],
                     "path_frac_of_burst": m["path_frac_of_burst"], "per_kernel_class": m["per_class"]},
        "cpu_baseline": cpu,
        "other_configs": others,
        "adjacent": adjacent,
    }
    print(json.dumps(out))


if __name__ == "__main__":
    main()

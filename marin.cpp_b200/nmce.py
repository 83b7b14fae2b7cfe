"""Host-side harness of libmarincpp_kernels.so for tests and benches: the nm_* entry points through ctypes, with torch
tensors supplying raw device pointers. It mirrors the reference's test harness (tests/s5/nmce.py:17-107: SIGS, Lib,
ptr, Ws, ce_call) so that tests written against the reference library read the same against this one. Torch is used
only for device memory and streams; every computation goes through the C ABI. There is no fallback: if the library is
missing or a call fails, an exception is raised.
"""
import ctypes
import os

C = ctypes
VP, I32, I64, U64, F32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmarincpp_kernels.so")

_CE_ARGS = [I32, I32, I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, I32, VP, VP, I32, I32, I64, I32, I32, I32, VP,
            VP]
SIGS = {
    "nm_version": (C.c_char_p, []),
    "nm_last_error": (C.c_char_p, []),
    "nm_device_arch": (I32, []),
    "nm_ce_workspace_bytes": (U64, [I32, I64, I32, I32, I32, I32]),
    "nm_fused_linear_ce": (I32, _CE_ARGS),
    "nm_fused_linear_ce_ex": (I32, _CE_ARGS + [F32, C.c_int32, VP]),
    "nm_ce_set_backends": (I32, [I32, I32, I32]),
    "nm_ce_set_fast_stats_exp": (I32, [I32]),
    "nm_ce_finish_microbatch": (I32, [VP, VP, I64, VP]),
    "nm_ce_grad_scale": (I32, [VP, I64, F32, VP, VP]),
    "nm_ce_readout": (I32, [I32, I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, VP, I32, VP, VP, VP, VP, VP, I32, I64, I32,
                            I32, I32, F32, VP, VP]),
    "nm_ce_dlogits": (I32, [I32, VP, I64, VP, VP, VP, I32, I32, VP]),
    "nm_ce_device_arch": (I32, []),
    "nm_ce_device_status": (I32, [VP, VP, VP]),
    "nm_ce_forward_noalloc": (I32, [VP, VP, VP, VP, VP, VP, VP, I64, I32, I32, I32, F32, C.c_int32, VP]),
    "nm_ce_profile_enable": (I32, [I32]),
    "nm_ce_profile_read": (I32, [VP, VP]),
    "nm_ce_test_wait_timeout": (I32, [VP, I64, VP, VP]),
    "nm_ce_set_cta_pair": (I32, [I32, I32, I32]),
    "nm_ce_suggest_chunk_rows": (I32, [I64]),
    "nm_ce_test_gemm": (I32, [I32, VP, I64, VP, I64, VP, I64, I32, I32, I32, VP, VP, VP]),
    "nm_ce_set_grad_path": (I32, [I32]),
    "nm_ce_set_tail_order": (I32, [I32]),
    "nm_ce_sampled_stride": (I64, [I64]),
    "nm_ce_sampled_workspace_bytes": (U64, [I64, I32, I32, I32, I32, I32]),
    "nm_ce_sampled_head": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, VP, I32, VP, I32, I64, I32, I32, I32, I64, I32,
                                 I32, VP, VP, VP, VP, F32, C.c_int32]),
    "nm_ce_forward_noalloc_status": (I32, [VP, VP]),
    "nm_ce_forward_noalloc_test_timeout": (I32, [I64, VP]),
    "nm_rmsnorm_fwd": (I32, [I32, I32, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_norm_partial_rows": (I64, [I64]),
    "nm_rmsnorm_bwd_add_partial": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_rmsnorm_bwd_add": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_sandwich_tail_fwd": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_sandwich_tail_bwd": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_doc_meta": (I32, [VP, VP, I32, I32, I32, I32, VP, VP, VP, VP, VP, VP, VP, VP]),
    "nm_sum_fixed": (I32, [VP, I64, VP, VP]),
    "nm_norm_bwd_device_status": (I32, [VP, VP]),
    "nm_norm_bwd_test_timeout": (I32, [I64, VP]),
    "nm_sandwich_tail_bwd_partial": (I32, [I32, I32, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, I64, I32, F32, VP]),
    "nm_reduce_partials_rows": (I32, [VP, I32, I32, VP, I32, I32, VP]),
    "nm_comm_unique_id": (I32, [VP]),
    "nm_comm_create": (I32, [VP, I32, I32, VP]),
    "nm_comm_destroy": (I32, [VP]),
    "nm_comm_allreduce_f32": (I32, [VP, VP, I64, VP]),
    "nm_grad_reducer_create": (I32, [VP, VP, I32, I32, I32, I32, VP, VP]),
    "nm_grad_bucket_ranges": (I32, [I32, I32, VP, VP, VP]),
    "nm_grad_reducer_destroy": (I32, [VP]),
    "nm_grad_reducer_reduce_all": (I32, [VP, VP]),
    "nm_grad_reducer_wait": (I32, [VP, VP]),
    "nm_adamh_update": (I32, [VP, VP, VP, VP, VP, I64, I64, I64, F32, F32, F32, F32, F32, I32, F32, VP, VP, VP, I32,
                              VP]),
    "nm_adam_update": (I32, [VP, VP, VP, VP, VP, I64, I64, I64, F32, F32, F32, F32, F32, I32, F32, VP, VP, VP, I32,
                             VP]),
    "nm_grad_reducer_create_owners": (I32, [VP, VP, I32, I32, I32, VP]),
    "nm_grad_reducer_owned_elems": (I64, [VP]),
    "nm_grad_reducer_microbatch_done": (I32, [VP, VP, VP]),
    "nm_grad_reducer_owned_to_grad": (I32, [VP, VP, VP]),
    "nm_head_adamh_create": (I32, [I32, I32, VP, VP]),
    "nm_head_adamh_destroy": (I32, [VP]),
    "nm_head_adamh_owned_elems": (I64, [VP]),
    "nm_head_adamh_ranges": (I32, [VP, I32, VP, VP, VP, VP]),
    "nm_head_adamh_init_master": (I32, [VP, VP, VP, VP]),
    "nm_head_adamh_step": (I32, [VP, I64, F32, F32, F32, F32, F32, F32, VP, VP, VP, VP, VP, VP]),
    "nm_head_adamh_step_async": (I32, [VP, I64, F32, F32, F32, F32, F32, F32, VP, VP, VP, VP, VP, VP]),
    "nm_head_adamh_wait_params": (I32, [VP, VP]),
    "nm_head_adamh_scalars": (I32, [VP, VP, VP]),
}
NO_STATUS = {"nm_version", "nm_last_error", "nm_device_arch", "nm_ce_workspace_bytes", "nm_ce_set_backends",
             "nm_ce_device_arch", "nm_ce_set_fast_stats_exp", "nm_ce_sampled_stride", "nm_ce_sampled_workspace_bytes", "nm_norm_partial_rows", "nm_head_adamh_owned_elems", "nm_grad_reducer_owned_elems", "nm_ce_suggest_chunk_rows"}

IMPLS = {"A": 0, "B1": 1, "B1.5": 2, "B2": 3}
LEV, ACC = 0, 1
F32S, BF16S = 0, 1


class NmError(RuntimeError):
    def __init__(self, name, status, message):
        super().__init__(f"{name} returned {status}: {message}")
        self.status = status


class Lib:
    """The shared library with typed entry points; a non-zero status raises NmError with nm_last_error()."""

    def __init__(self, path=None):
        path = path or LIB_PATH
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: build it with `python marin.cpp_b200/build.py` (no fallback)")
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in SIGS.items():
            f = getattr(self.dll, name)
            f.restype, f.argtypes = res, args

    def raw(self, name):
        return getattr(self.dll, name)

    def __getattr__(self, name):
        f = getattr(self.dll, name)

        def call(*a):
            r = f(*a)
            if name not in NO_STATUS and r != 0:
                raise NmError(name, r, self.dll.nm_last_error().decode())
            return r
        return call


def ptr(t):
    """Device (or host) pointer of a torch tensor / numpy array, None for None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return VP(t.data_ptr())
    return VP(t.ctypes.data)


class Ws:
    """One CE workspace, grown on demand (torch's allocator; 256-byte aligned by construction)."""
    buf = None

    @classmethod
    def get(cls, nbytes, device="cuda"):
        import torch
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        if cls.buf is None or cls.buf.numel() < nbytes or cls.buf.device != device:
            cls.buf = None
            torch.cuda.empty_cache()
            cls.buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        return cls.buf


def ce_call(lib, impl, x, W, targets, weight, gscale, *, rounding=LEV, store=BF16S, chunk=1024, dx=None, acc_dx=False,
            dw=None, dw_mb=None, dw_round=0, forward_only=False, bias=None, loss_partial=None, lse=None, io=None,
            ws=None, z_loss=None, ignore_index=None, reducer=None, stream=None, loss=None, check=True):
    """Runs nm_fused_linear_ce (or the _ex entry point when z_loss / ignore_index / reducer is given). Returns
    (loss_tok, lse). dx / dw / dw_mb are written in place. check: synchronise and read the device status word."""
    import torch
    T, D = x.shape
    V = W.shape[0]
    io = (0 if x.dtype == torch.float32 else 1) if io is None else io
    dev = x.device
    loss = torch.empty(T, dtype=torch.float32, device=dev) if loss is None else loss
    lse = torch.empty(T, dtype=torch.float32, device=dev) if lse is None else lse
    if ws is None:
        ws = Ws.get(lib.nm_ce_workspace_bytes(IMPLS[impl], T, D, V, chunk, store), dev)
    st = None if stream is None else VP(stream)
    args = [IMPLS[impl], rounding, io, store, ptr(x), ptr(W), ptr(targets), ptr(weight), ptr(gscale), ptr(bias),
            ptr(loss), ptr(lse), ptr(loss_partial), ptr(dx), int(acc_dx), ptr(dw), ptr(dw_mb), dw_round,
            int(forward_only), T, D, V, chunk, ptr(ws), st]
    if z_loss is None and ignore_index is None and reducer is None:
        lib.nm_fused_linear_ce(*args)
    else:
        lib.nm_fused_linear_ce_ex(*args, 0.0 if z_loss is None else float(z_loss),
                                  -2 ** 31 if ignore_index is None else int(ignore_index), reducer)
    if check and T > 0:
        status = C.c_uint32(0)
        lib.nm_ce_device_status(ptr(ws), st, C.byref(status))
    return loss, lse

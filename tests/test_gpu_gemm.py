"""The three tcgen05 contractions alone (nm_ce_test_gemm) against a float32 torch reference of the same product of
bf16 operands: K-major x K-major (logits), K-major x MN-major (dX), MN-major x MN-major (dW); full, ragged and
single-tile shapes; one CTA per tile (kinds 0-2) and a pair of CTAs per tile (kinds 4-6). Tolerance: f32 accumulation of exactly representable bf16 products, so relative L2 <= 1e-5."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 768, 1024), (304, 520, 200), (8, 8, 8),
          (1, 16, 72), (1000, 264, 136), (2048, 2048, 4096)]


@pytest.mark.parametrize("kind", [0, 1, 2, 4, 5, 6])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_umma_contraction(kind, M, N, K):
    from gpu_common import lib, nmce, rel
    kind_arg, kind = kind, kind & 3
    if kind == 2 and M % 8:
        M = (M + 7) // 8 * 8          # an MN-major A has M contiguous: its row pitch must be a multiple of 16 bytes
    g = torch.Generator(device="cuda").manual_seed(1000 * kind + M + N + K)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    B = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    want = A.float() @ B.float().T
    if kind == 0:
        a, lda, b, ldb = A, K, B, K
    elif kind == 1:
        a, lda, b, ldb = A, K, B.T.contiguous(), N          # B stored [K, N]
    else:
        a, lda, b, ldb = A.T.contiguous(), M, B.T.contiguous(), N   # A stored [K, M]
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib().nm_ce_test_gemm(kind_arg, nmce.ptr(a), lda, nmce.ptr(b), ldb, nmce.ptr(c), N, M, N, K, nmce.ptr(status), None)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"a bounded device wait ran out: status {int(status.item())}"
    assert torch.isfinite(c).all(), "the kernel left part of C unwritten"
    r = rel(c, want)
    assert r <= 1e-5, f"kind {kind_arg} M{M} N{N} K{K}: rel {r:.3e}"

"""The tcgen05 contractions alone (nm_ce_test_gemm) against a float32 torch reference of the same product of
bf16 operands: K-major x K-major (logits), K-major x MN-major (dX), MN-major x MN-major (dW); full, ragged and
single-tile shapes; one CTA per tile (kinds 0-2), a pair of CTAs per tile (kinds 4-6), and the pair kernels with one
512-column accumulator (kinds 9, 10), also with the A operand given as raw logits that the kernel turns into the
normalised gradient in shared memory (kinds 25, 26). Tolerance: f32 accumulation of exactly representable bf16
products, so relative L2 <= 1e-5."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 768, 1024), (304, 520, 200), (8, 8, 8),
          (1, 16, 72), (1000, 264, 136), (2048, 2048, 4096)]


@pytest.mark.parametrize("kind", [0, 1, 2, 4, 5, 6, 9, 10])
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
    lib().nm_ce_test_gemm(kind_arg, nmce.ptr(a), lda, nmce.ptr(b), ldb, nmce.ptr(c), N, M, N, K, nmce.ptr(status), None,
                          None)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"a bounded device wait ran out: status {int(status.item())}"
    assert torch.isfinite(c).all(), "the kernel left part of C unwritten"
    r = rel(c, want)
    assert r <= 1e-5, f"kind {kind_arg} M{M} N{N} K{K}: rel {r:.3e}"


WIDE_SHAPES = [(256, 512, 64), (256, 512, 512), (512, 1024, 256), (304, 520, 200), (8, 8, 8), (1000, 264, 136),
               (2048, 512, 4096), (1280, 2048, 1000)]


@pytest.mark.parametrize("kind", [25, 26])
@pytest.mark.parametrize("M,N,K", WIDE_SHAPES)
def test_wide_contraction_forms_the_gradient_on_the_fly(kind, M, N, K):
    """A holds raw bf16 logits z; the kernel must contract n = bf16(a p - b onehot(target)), p = 2^(z log2e + e), with
    B, where (e, a, b, target) are per row of the logits matrix: the M rows for kind 25 (the dX layout: logits [M, K],
    K = vocabulary), the K rows for kind 26 (the dW layout: logits [K, M], M = vocabulary). The expected n is formed in
    torch with the same roundings (f32 product and difference, one rounding to bf16), up to the 2-ulp ex2.approx:
    against that, the product is held to 2e-3 relative (measured ~1e-3: an ulp of bf16 n where p differs in the last
    f32 bits), and columns of the logits at or beyond the vocabulary must contribute nothing."""
    from gpu_common import lib, nmce, rel
    k = kind & 3
    if k == 2 and M % 8:
        M = (M + 7) // 8 * 8
    g = torch.Generator(device="cuda").manual_seed(77 * kind + M + N + K)
    rows, vocab = (M, K) if k == 1 else (K, M)           # shape of the logits matrix
    ld = (vocab + 7) // 8 * 8                             # the store's row pitch: a multiple of 8, padding is garbage
    Z = torch.full((rows, ld), float("nan"), dtype=torch.bfloat16, device="cuda")
    Z[:, :vocab] = (torch.randn(rows, vocab, generator=g, device="cuda") * 1.5).to(torch.bfloat16)
    lse = torch.logsumexp(Z[:, :vocab].float(), dim=1) + 0.3 * torch.randn(rows, generator=g, device="cuda")
    a = torch.rand(rows, generator=g, device="cuda") + 0.5
    b = torch.rand(rows, generator=g, device="cuda") + 0.5
    tg = torch.randint(0, vocab, (rows,), generator=g, device="cuda", dtype=torch.int32)
    a[::5] = 0
    b[::5] = 0                                            # ignored rows
    tg[::5] = -1
    e = -lse * 1.4426950408889634
    rf = torch.empty(rows, 4, dtype=torch.float32, device="cuda")
    rf[:, 0], rf[:, 1], rf[:, 2] = e, a, b
    rf[:, 3] = tg.view(torch.float32)
    n = torch.exp2(Z[:, :vocab].float() * 1.4426950408889634 + e[:, None]) * a[:, None]
    hit = tg >= 0
    n[torch.arange(rows, device="cuda")[hit], tg[hit].long()] -= b[hit]
    n = n.to(torch.bfloat16).float()
    B = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    Bs = B.T.contiguous()                                 # stored [K, N]
    if k == 1:
        want = n @ B.float().T                            # [M, N], contraction over the vocabulary
        a_arg, lda = Z, ld
    else:
        want = n.T @ B.float().T                          # [M = vocabulary, N], contraction over the rows
        a_arg, lda = Z, ld                                # A stored [K, M]: the logits as they are
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib().nm_ce_test_gemm(kind, nmce.ptr(a_arg), lda, nmce.ptr(Bs), N, nmce.ptr(c), N, M, N, K, nmce.ptr(status),
                          nmce.ptr(rf), None)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"a bounded device wait ran out: status {int(status.item())}"
    assert torch.isfinite(c).all(), "the kernel left part of C unwritten, or garbage columns leaked in"
    r = rel(c, want)
    assert r <= 2e-3, f"kind {kind} M{M} N{N} K{K}: rel {r:.3e}"

"""The split-fp32 tensor-core product against an fp64 product (floating point: tolerance stated)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# Relative Frobenius error allowed.  Three tf32 products of a hi/lo split keep ~2^-21 per
# term; the tensor core's accumulator truncates (about 7e-9 of the sum per element of k), which
# the kernel lets run up to k = 512 and confines to chunks of 128 beyond that (the chunks are
# summed with rounding), so the error must not grow with k.
TOL = 2.5e-6


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (128, 128, 128), (256, 384, 512), (200, 132, 72),
                                   (1000, 520, 264), (4096, 1024, 128), (130, 4096, 128),
                                   (512, 384, 4096), (256, 256, 11008)])
@pytest.mark.parametrize("b_is_kn", [False, True])
def test_gemm_matches_fp64(dgq, m, n, k, b_is_kn):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g, device="cuda")
    b = torch.randn((k, n) if b_is_kn else (n, k), generator=g, device="cuda")
    c0 = torch.randn(m, n, generator=g, device="cuda")
    want = -0.5 * (a.double() @ (b.double() if b_is_kn else b.double().t())) + 2.0 * c0.double()
    c = c0.clone()
    info = dgq.new_info("cuda")
    dgq.gemm_f32(a, b, c, b_is_kn, alpha=-0.5, beta=2.0, info=info)
    dgq.raise_on_info(info, "gemm")
    assert _rel(c, want) <= TOL
    ref32 = -0.5 * (a @ (b if b_is_kn else b.t())) + 2.0 * c0
    assert _rel(c, want) <= 20 * max(_rel(ref32, want), 1e-8)
    if k >= 4096:       # long reductions: as accurate as torch's fp32 product, within a small factor
        assert _rel(c, want) <= 3 * _rel(ref32, want)
    # beta = 0 must not read C (NaNs in C stay out of the result)
    c = torch.full((m, n), float("nan"), device="cuda")
    dgq.gemm_f32(a, b, c, b_is_kn)
    assert _rel(c, a.double() @ (b.double() if b_is_kn else b.double().t())) <= TOL


def test_gemm_strided_views_and_lower_only(dgq):
    g = torch.Generator(device="cuda").manual_seed(5)
    big = torch.randn(700, 900, generator=g, device="cuda")
    a = big[64:64 + 300, 128:128 + 260]            # offsets keep 16-byte alignment
    bt = big[400:400 + 300, 256:256 + 260]
    cbuf = torch.zeros(320, 400, device="cuda")
    c = cbuf[:300, 64:64 + 300]
    dgq.gemm_f32(a, bt, c, False, alpha=1.0, beta=0.0, lower_only=True)
    want = torch.tril(a.double() @ bt.double().t())
    assert _rel(c, want) <= TOL
    assert float(torch.triu(c, 1).abs().max()) == 0          # nothing written above the diagonal
    assert float(cbuf[300:].abs().max()) == 0 and float(cbuf[:, :64].abs().max()) == 0
    assert float(cbuf[:, 364:].abs().max()) == 0


def test_gemm_rejects_misaligned(dgq):
    a = torch.zeros(128, 130, device="cuda")[:, 1:129]
    b = torch.zeros(128, 128, device="cuda")
    c = torch.zeros(128, 128, device="cuda")
    with pytest.raises(RuntimeError, match="align"):
        dgq.gemm_f32(a, b, c, False)

"""Hessian accumulation (tcgen05 kernel) against the oracle / the reference's add_batch."""
import pytest
import torch

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def rel_fro(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _x(Tk, K, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Tk, K, generator=g)
    if outliers:
        idx = torch.randperm(K, generator=g)[:max(1, K // 100)]
        x[:, idx] *= 20
    return x.bfloat16()


@pytest.mark.parametrize("Tk,K", [(64, 64), (100, 8), (128, 256), (1000, 320), (4096, 768),
                                  (777, 1032), (2048, 2048)])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_hessian_matches_oracle(dgq, Tk, K, splits):
    x = _x(Tk, K, Tk + K)
    want, _ = O.hessian_add_batch(None, 0, x.float())
    H = torch.zeros((K, K), dtype=torch.float32, device="cuda")
    info = dgq.new_info("cuda")
    dgq.hessian_accum(x.cuda(), H, 1.0, splits, info)
    dgq.raise_on_info(info, "hessian")
    assert rel_fro(H.cpu(), want) <= 1e-3        # the stated tolerance
    assert rel_fro(H.cpu(), want) <= 5e-5        # what fp32 accumulation of exact products gives
    if splits == 1:
        assert torch.equal(H, H.t())             # both triangles receive the same values
    else:
        # token ranges add into H in no fixed order, so the triangles agree to rounding only
        assert rel_fro(H, H.t()) <= 1e-6


def test_hessian_accumulates_and_scales(dgq):
    K = 512
    xs = [_x(300 + 50 * i, K, i) for i in range(3)]
    want = None
    n = 0
    for x in xs:
        want, n = O.hessian_add_batch(want, n, x.float())
    H = torch.zeros((K, K), dtype=torch.float32, device="cuda")
    for x in xs:
        dgq.hessian_accum(x.cuda(), H)
    assert rel_fro(H.cpu(), want) <= 2e-6
    H2 = torch.zeros_like(H)
    dgq.hessian_accum(xs[0].cuda(), H2, alpha=0.5)
    w0, _ = O.hessian_add_batch(None, 0, xs[0].float())
    assert rel_fro(H2.cpu(), 0.5 * w0) <= 2e-6


def test_hessian_deterministic_without_splits(dgq):
    x = _x(3000, 1024, 5).cuda()
    a = torch.zeros((1024, 1024), dtype=torch.float32, device="cuda")
    b = torch.zeros_like(a)
    dgq.hessian_accum(x, a, 1.0, 1)
    dgq.hessian_accum(x, b, 1.0, 1)
    assert torch.equal(a, b)


def test_hessian_strided_views(dgq):
    # X a column slice of a wider buffer, H a window of a padded buffer
    big = _x(500, 1024, 9).cuda()
    x = big[:, 256:256 + 384]
    Hbuf = torch.zeros((400, 400), dtype=torch.float32, device="cuda")
    H = Hbuf[:384, :384]
    dgq.hessian_accum(x, H)
    want, _ = O.hessian_add_batch(None, 0, x.float().cpu())
    assert rel_fro(H.cpu(), want) <= 2e-6
    assert float(Hbuf[384:].abs().max()) == 0 and float(Hbuf[:, 384:].abs().max()) == 0


def test_gptq_add_batch_matches_reference_golden(dgq, ref_pins):
    import torch.nn as nn
    from distributed_gptq_b200 import GPTQ
    p = ref_pins
    lin = nn.Linear(24, 16, bias=False).cuda()
    q = GPTQ(lin, bits=4, group_size=8, blocksize=8)
    # golden inputs are fp32: the kernel rounds them to bf16, so compare at the stated tolerance
    q.add_batch(T(p["ab_x3"]).cuda(), None)
    assert q.nsamples == int(p["ab_n1"]) and q.H.shape == (24, 24) and q.H.dtype == torch.float32
    assert rel_fro(q.H.cpu(), T(p["ab_H1"])) <= 1e-2
    q.add_batch(T(p["ab_x2"]).cuda(), None)
    assert q.nsamples == int(p["ab_n2"])
    assert rel_fro(q.H.cpu(), T(p["ab_H2"])) <= 1e-2
    # bf16 activations: products are exact, fp32 accumulation
    q2 = GPTQ(nn.Linear(24, 16, bias=False).cuda())
    q2.add_batch(T(p["ab_xb"]).reshape(2, 12, 24).bfloat16().cuda(), None)
    assert rel_fro(q2.H.cpu(), T(p["ab_Hb"])) <= 2e-6


def test_hessian_layer_sweep_shape_property(dgq):
    # K = 4096 at a reduced token count: symmetric, PSD diagonal, matches fp32 matmul on device
    K, Tk = 4096, 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(Tk, K, generator=g, device="cuda").bfloat16()
    H = torch.zeros((K, K), dtype=torch.float32, device="cuda")
    dgq.hessian_accum(x, H)
    ref = x.float().t() @ x.float()
    assert rel_fro(H, ref) <= 1e-3
    assert rel_fro(H, H.t()) <= 1e-6


def test_rejects_bad_arguments(dgq):
    x = torch.zeros((64, 12), dtype=torch.bfloat16, device="cuda")   # K not a multiple of 8
    H = torch.zeros((12, 12), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="align"):
        dgq.hessian_accum(x, H)


def test_upper_only_accumulation_and_mirror(dgq):
    """`dgq_hessian_accum_upper` over several batches followed by one `dgq_hessian_mirror` gives
    the matrix `dgq_hessian_accum` builds, bit for bit (one token range per launch, so every
    element receives the same additions in the same order)."""
    g = torch.Generator(device="cuda").manual_seed(4)
    for K in (264, 1024):
        full = torch.zeros(K, K, device="cuda")
        upper = torch.full((K, K), 7.0, device="cuda").tril(-1)      # junk below the diagonal
        for _ in range(3):
            x = torch.randn(2048, K, generator=g, device="cuda").bfloat16()
            dgq.hessian_accum(x, full, 1.0, 1)
            dgq.hessian_accum(x, upper, 1.0, 1, upper_only=True)
        assert torch.equal(upper.tril(-1), torch.full((K, K), 7.0, device="cuda").tril(-1))
        dgq.hessian_mirror(upper)
        assert torch.equal(upper, full) and torch.equal(upper, upper.t())


def test_long_accumulation_chains_stay_inside_the_bar(dgq):
    """The tensor core's fp32 accumulator truncates, so the error of one launch grows with the
    tokens it carries (one token range = one accumulation chain).  65536 tokens in one range is
    what the model driver feeds per call; the result must stay well inside the 1e-3 bar, and
    cutting the range (`splits`) must shrink the error in proportion."""
    K, T = 1024, 65536
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(T, K, generator=g, device="cuda")
    x[:, ::97] *= 20
    xb = x.bfloat16()
    want = xb.double().t() @ xb.double()
    errs = {}
    for splits in (1, 4):
        H = torch.zeros(K, K, device="cuda")
        dgq.hessian_accum(xb, H, 1.0, splits)
        errs[splits] = float((H.double() - want).norm() / want.norm())
    assert errs[1] <= 5e-4, errs
    assert errs[4] <= 0.4 * errs[1], errs

"""dgq_qlinear_forward against the oracle's dequantize + matmul."""
import pytest
import torch

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 2, 4, 7, 16, 33])
@pytest.mark.parametrize("N_out,K,g,bits", [(64, 128, 32, 4), (100, 520, 128, 4), (37, 203, 64, 4),
                                             (256, 1024, 128, 8), (64, 256, 64, 3), (48, 512, -1, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_qlinear(dgq, M, N_out, K, g, bits, dtype):
    gen = torch.Generator().manual_seed(M * 7 + N_out + K)
    codes = torch.randint(0, 2 ** bits, (N_out, K), generator=gen).to(torch.uint8)
    ng = O.n_groups(K, g)
    scales = (torch.rand(N_out, ng, generator=gen) * 0.02 + 0.001).half()
    zeros = torch.randint(0, 2 ** bits, (N_out, ng), generator=gen).half()
    gg = K if g <= 0 else g
    g_idx = (torch.arange(K) // gg).to(torch.int32)
    g_idx = g_idx[torch.randperm(K, generator=gen)]            # act-order style mapping
    bias = torch.randn(N_out, generator=gen).to(dtype)
    x = torch.randn(M, K, generator=gen).to(dtype)
    qw = O.pack_f2(codes, bits)
    want = O.qlinear_forward(x, codes, scales, zeros, g_idx, bias, g)
    got = dgq.qlinear_forward(x.cuda(), qw.cuda(), scales.cuda(), zeros.cuda(), g_idx.cuda(),
                              bias.cuda(), K, bits, g)
    assert got.dtype == dtype and tuple(got.shape) == (M, N_out)
    tol = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    scale = want.abs().max()
    assert float((got.float().cpu() - want).abs().max()) <= tol * float(scale)
    # no g_idx, no bias
    want2 = O.qlinear_forward(x, codes, scales, zeros, None, None, g)
    got2 = dgq.qlinear_forward(x.cuda(), qw.cuda(), scales.cuda(), zeros.cuda(), None, None, K, bits, g)
    assert float((got2.float().cpu() - want2).abs().max()) <= tol * float(want2.abs().max())


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33])
@pytest.mark.parametrize("N_out,K,g", [(64, 128, 128), (100, 512, 128), (37, 1024, 256), (256, 384, -1),
                                       (1000, 2048, 128)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("integer_zeros", [True, False])
def test_qlinear_tensor_core_path(dgq, M, N_out, K, g, dtype, integer_zeros):
    """4-bit codes, 16-bit activations, whole groups of 128 columns, no g_idx: the warp-level
    multiply-accumulate kernel.  Products are exact and accumulate in fp32, so the only rounding
    is the output's (and, for fractional zero points, the 16-bit subtraction)."""
    gen = torch.Generator().manual_seed(M * 11 + N_out + K)
    codes = torch.randint(0, 16, (N_out, K), generator=gen).to(torch.uint8)
    ng = O.n_groups(K, g)
    scales = (torch.rand(N_out, ng, generator=gen) * 0.02 + 0.001).half()
    if integer_zeros:
        zeros = torch.randint(0, 16, (N_out, ng), generator=gen).half()
    else:
        zeros = (torch.rand(N_out, ng, generator=gen) * 15).half()
    bias = torch.randn(N_out, generator=gen).to(dtype)
    x = torch.randn(M, K, generator=gen).to(dtype)
    qw = O.pack_f2(codes, 4)
    want = O.qlinear_forward(x, codes, scales, zeros, None, bias, g)
    got = dgq.qlinear_forward(x.cuda(), qw.cuda(), scales.cuda(), zeros.cuda(), None, bias.cuda(), K, 4, g)
    assert got.dtype == dtype and tuple(got.shape) == (M, N_out)
    tol = {torch.float16: 6e-4, torch.bfloat16: 4.5e-3}[dtype]
    if not integer_zeros:
        tol *= 2
    assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("M", [1, 5, 16, 40])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_operator_with_act_order_checkpoint(dgq, M, dtype):
    """An act-order checkpoint through ``torch.ops.gptq.linear``: the group of a column is
    arbitrary (every group still has 128 columns).  The operator brings the columns into group
    order once and gathers the activations per call, so the result must be that of the
    dequantize + matmul of models/layers.py:155-157 to the kernel's tolerance, call after call."""
    import distributed_gptq_b200  # noqa: F401
    N_out, K, g = 320, 1024, 128
    gen = torch.Generator().manual_seed(M)
    codes = torch.randint(0, 16, (N_out, K), generator=gen).to(torch.uint8)
    scales = (torch.rand(N_out, K // g, generator=gen) * 0.02 + 0.001).half()
    zeros = torch.randint(0, 16, (N_out, K // g), generator=gen).half()
    g_idx = (torch.arange(K) // g).to(torch.int32)[torch.randperm(K, generator=gen)]
    bias = torch.randn(N_out, generator=gen).to(dtype)
    x = torch.randn(2, M, K, generator=gen).to(dtype)
    want = O.qlinear_forward(x.reshape(-1, K), codes, scales, zeros, g_idx, bias, g).reshape(2, M, N_out)
    qw, s, z, gi, b = (t.cuda() for t in (O.pack_f2(codes, 4), scales, zeros, g_idx, bias))
    n0 = dgq.launch_count()
    for _ in range(2):      # the second call finds the reordered weights on the buffer
        got = torch.ops.gptq.linear(x.cuda(), qw, s, z, gi, b)
        assert got.dtype == dtype and tuple(got.shape) == (2, M, N_out)
        tol = {torch.float16: 6e-4, torch.bfloat16: 4.5e-3}[dtype]
        assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    assert hasattr(qw, "_dgq_grouped") and dgq.launch_count() > n0
    # uneven groups cannot be reordered into whole groups: the general kernel takes them
    odd = g_idx.clone()
    odd[odd == 1] = 0
    want2 = O.qlinear_forward(x.reshape(-1, K), codes, scales, zeros, odd, bias, g).reshape(2, M, N_out)
    got2 = torch.ops.gptq.linear(x.cuda(), qw.clone(), s, z, odd.cuda(), b)
    tol = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    assert float((got2.float().cpu() - want2).abs().max()) <= tol * float(want2.abs().max())


@pytest.mark.parametrize("M", [33, 64, 200, 256, 1000])
@pytest.mark.parametrize("N_out,K,g", [(256, 512, 128), (1000, 2048, 128), (320, 1024, 64),
                                       (128, 256, -1), (136, 4096, 256)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qlinear_many_rows(dgq, M, N_out, K, g, dtype):
    """More than 32 rows of activations: the tcgen05 kernel that dequantizes the weights into
    shared memory (one rounding of (code - zero) * scale to the activation type, exact
    products, fp32 accumulation), against dequantize + matmul (models/layers.py:155-157)."""
    gen = torch.Generator().manual_seed(M + N_out + K)
    codes = torch.randint(0, 16, (N_out, K), generator=gen).to(torch.uint8)
    ng = O.n_groups(K, g)
    scales = (torch.rand(N_out, ng, generator=gen) * 0.02 + 0.001).half()
    zeros = torch.randint(0, 16, (N_out, ng), generator=gen).half()
    bias = torch.randn(N_out, generator=gen).to(dtype)
    x = torch.randn(M, K, generator=gen).to(dtype)
    qw = O.pack_f2(codes, 4)
    want = O.qlinear_forward(x, codes, scales, zeros, None, bias, g)
    n0 = dgq.launch_count()
    got = dgq.qlinear_forward(x.cuda(), qw.cuda(), scales.cuda(), zeros.cuda(), None, bias.cuda(), K, 4, g)
    assert dgq.launch_count() == n0 + 1            # one launch for all rows
    assert got.dtype == dtype and tuple(got.shape) == (M, N_out)
    tol = {torch.float16: 8e-4, torch.bfloat16: 6e-3}[dtype]
    assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    # without bias, and checked against the product with the weights rounded as the kernel rounds them
    got2 = dgq.qlinear_forward(x.cuda(), qw.cuda(), scales.cuda(), zeros.cuda(), None, None, K, 4, g)
    Wt = O.dequant(codes, scales, zeros, None, g).to(dtype).double()
    exact = (x.double() @ Wt.t())
    out_eps = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[dtype]
    assert float((got2.double().cpu() - exact).abs().max()) <= 1.01 * out_eps * float(exact.abs().max()) + 1e-6


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("g", [128, 64])
def test_qlinear_prefill_sized(dgq, dtype, g):
    """Enough 256 x 256 tiles for several rounds on every SM: the kernel takes its largest
    tile (one set of accumulators, one converter group), with ragged edges in both
    directions.  Checked on a sample of rows (rows are independent)."""
    M, N_out, K = 4100, 9608, 512
    assert -(-M // 256) * -(-N_out // 256) >= 4 * torch.cuda.get_device_properties(0).multi_processor_count
    gen = torch.Generator().manual_seed(11)
    codes = torch.randint(0, 16, (N_out, K), generator=gen).to(torch.uint8)
    ng = O.n_groups(K, g)
    scales = (torch.rand(N_out, ng, generator=gen) * 0.02 + 0.001).half()
    zeros = torch.randint(0, 16, (N_out, ng), generator=gen).half()
    bias = torch.randn(N_out, generator=gen).to(dtype)
    x = torch.randn(M, K, generator=gen).to(dtype)
    n0 = dgq.launch_count()
    got = dgq.qlinear_forward(x.cuda(), O.pack_f2(codes, 4).cuda(), scales.cuda(), zeros.cuda(), None,
                              bias.cuda(), K, 4, g)
    assert dgq.launch_count() == n0 + 1 and tuple(got.shape) == (M, N_out)
    rows = torch.cat([torch.arange(0, 8), torch.randint(0, M, (240,), generator=gen),
                      torch.arange(M - 8, M)])
    Wt = O.dequant(codes, scales, zeros, None, g).to(dtype).double()
    exact = x[rows].double() @ Wt.t() + bias.double()
    out_eps = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[dtype]
    err = (got[rows.cuda()].double().cpu() - exact).abs().max()
    assert float(err) <= 1.01 * out_eps * float(exact.abs().max()) + 1e-6
    # the other rows: finite, and consistent with the sampled ones in magnitude
    assert bool(torch.isfinite(got).all())
    assert float(got.float().abs().max()) <= 1.5 * float(exact.abs().max()) + 1.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qlinear_many_rows_fractional_zero_points(dgq, dtype):
    """Zero points that are not integers (the flat round-to-nearest helpers produce them) take the
    kernel's fp32 dequantization instead of the two-instruction one."""
    M, N_out, K, g = 96, 200, 768, 128
    gen = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 16, (N_out, K), generator=gen).to(torch.uint8)
    scales = (torch.rand(N_out, K // g, generator=gen) * 0.02 + 0.001).half()
    zeros = (torch.rand(N_out, K // g, generator=gen) * 15).half()
    zeros[::2] = zeros[::2].round()              # both kinds within one tile
    x = torch.randn(M, K, generator=gen).to(dtype)
    want = O.qlinear_forward(x, codes, scales, zeros, None, None, g)
    got = dgq.qlinear_forward(x.cuda(), O.pack_f2(codes, 4).cuda(), scales.cuda(), zeros.cuda(), None,
                              None, K, 4, g)
    tol = {torch.float16: 8e-4, torch.bfloat16: 6e-3}[dtype]
    assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())

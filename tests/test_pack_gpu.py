"""pack / unpack / unpack+dequant / scale-zero / RTN kernels against the oracle: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def _codes(rows, cols, bits, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 2 ** bits, (rows, cols), generator=g).to(torch.uint8)


SHAPES_ANY = [(1, 1), (3, 7), (5, 27), (6, 32), (16, 40), (9, 333), (33, 1280), (64, 4096)]


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("fmt", [1, 2, 3])
@pytest.mark.parametrize("shape", SHAPES_ANY)
def test_pack_unpack_bit_exact(dgq, bits, fmt, shape):
    rows, cols = shape
    if fmt == 1 and ((bits == 4 and cols % 2) or (bits == 2 and cols % 4)):
        pytest.skip("format 1 needs whole bytes")
    codes = _codes(rows, cols, bits, bits * 1000 + fmt * 100 + cols)
    want = O.pack(codes, bits, fmt)
    got = dgq.pack(codes.cuda(), bits, fmt)
    assert got.dtype == want.dtype and tuple(got.shape) == tuple(want.shape)
    assert torch.equal(got.cpu(), want)
    back = dgq.unpack(got, cols, bits, fmt)
    assert torch.equal(back.cpu(), codes)


def test_pack_matches_reference_golden(dgq, ref_pins):
    for bits in (2, 3, 4, 8):
        codes = T(ref_pins[f"f1_codes_{bits}"]).cuda()
        got = dgq.pack(codes, bits, dgq.FMT_BYTES_HI_FIRST).cpu().numpy()
        assert np.array_equal(got, ref_pins[f"f1_packed_{bits}"])
    for tag in ("even", "odd"):
        for bits in (3, 4, 8):
            codes = T(ref_pins[f"f2_{tag}_codes_{bits}"]).cuda()
            got = dgq.pack(codes, bits, dgq.FMT_BYTES_LO_FIRST).cpu().numpy()
            assert np.array_equal(got, ref_pins[f"f2_{tag}_qweight_{bits}"])
            deq = dgq.unpack_dequant(T(ref_pins[f"f2_{tag}_qweight_{bits}"]).cuda(),
                                     T(ref_pins[f"f2_{tag}_scales_{bits}"]).cuda(),
                                     T(ref_pins[f"f2_{tag}_zeros_{bits}"]).cuda(), None,
                                     codes.shape[1], bits, int(ref_pins["f2_group_size"]),
                                     dgq.FMT_BYTES_LO_FIRST)
            assert np.array_equal(deq.cpu().numpy(), ref_pins[f"f2_{tag}_deq_{bits}"])


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("fmt", [1, 2, 3])
@pytest.mark.parametrize("shape,g", [((5, 27), 8), ((7, 64), 16), ((33, 1280), 128), ((8, 4096), 128),
                                     ((4, 512), -1)])
@pytest.mark.parametrize("use_gidx", [False, True])
def test_unpack_dequant(dgq, bits, fmt, shape, g, use_gidx):
    rows, cols = shape
    if fmt == 1 and ((bits == 4 and cols % 2) or (bits == 2 and cols % 4)):
        pytest.skip("format 1 needs whole bytes")
    gen = torch.Generator().manual_seed(cols + bits)
    codes = _codes(rows, cols, bits, 77 + cols)
    ng = O.n_groups(cols, g)
    scales = (torch.rand(rows, ng, generator=gen) * 0.05 + 0.001)
    zeros = torch.randint(0, 2 ** bits, (rows, ng), generator=gen).float()
    g_idx = None
    if use_gidx:
        g_idx = torch.randint(0, ng, (cols,), generator=gen).to(torch.int32)
    packed = O.pack(codes, bits, fmt).cuda()
    for pdt in (torch.float32, torch.float16):
        s, z = scales.to(pdt), zeros.to(pdt)
        want = O.dequant(codes, s, z, g_idx, g)
        got = dgq.unpack_dequant(packed, s.cuda(), z.cuda(), None if g_idx is None else g_idx.cuda(),
                                 cols, bits, g, fmt, torch.float32)
        assert torch.equal(got.cpu(), want)
        for odt in (torch.bfloat16, torch.float16):
            got = dgq.unpack_dequant(packed, s.cuda(), z.cuda(),
                                     None if g_idx is None else g_idx.cuda(), cols, bits, g, fmt, odt)
            assert torch.equal(got.cpu(), want.to(odt))


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_find_params_and_quantize_rows(dgq, ref_pins, bits):
    wg = T(ref_pins[f"sf_wgroup_{bits}"])
    s, z = dgq.find_params(wg.cuda(), bits)
    assert torch.equal(s.cpu(), T(ref_pins[f"sf_scale_{bits}"]))
    assert torch.equal(z.cpu(), T(ref_pins[f"sf_zero_{bits}"]))
    q, xh = dgq.quantize_rows(wg[:, 3:4].contiguous().cuda(), s, z, bits)
    assert torch.equal(q.cpu().float().flatten(), T(ref_pins[f"sf_q_{bits}"]))
    assert torch.equal(xh.cpu().flatten(), T(ref_pins[f"sf_what_{bits}"]))
    # larger random case, incl. a constant row (scale falls back to 1)
    gen = torch.Generator().manual_seed(bits)
    x = torch.randn(257, 300, generator=gen) * 0.02
    x[5] = 0.125
    so, zo = O.find_params(x, 2 ** bits - 1)
    s, z = dgq.find_params(x.cuda(), bits)
    assert torch.equal(s.cpu(), so) and torch.equal(z.cpu(), zo)
    q, xh = dgq.quantize_rows(x.cuda(), s, z, bits)
    qo = torch.clamp(torch.round(x / so[:, None] + zo[:, None]), 0, 2 ** bits - 1)
    assert torch.equal(q.cpu().float(), qo)
    assert torch.equal(xh.cpu(), (qo - zo[:, None]) * so[:, None])


@pytest.mark.parametrize("bits,g,shape", [(4, 128, (64, 256)), (3, 64, (7, 100)), (8, 32, (1000,)),
                                          (2, 128, (5, 5, 31))])
def test_rtn(dgq, bits, g, shape):
    gen = torch.Generator().manual_seed(bits + g)
    x = torch.randn(*shape, generator=gen)
    qo, so, zo = O.rtn_quantize(x, bits, g)
    s, z = dgq.rtn_find_params(x.cuda(), bits, g)
    assert torch.equal(s.cpu(), so) and torch.equal(z.cpu(), zo)
    q = dgq.rtn_quantize(x.cuda(), s, z, bits, g)
    assert torch.equal(q.cpu(), qo)
    d = dgq.rtn_dequantize(q, s, z, g)
    assert torch.equal(d.cpu(), O.rtn_dequantize(qo, so, zo, g))


def test_large_round_trip_property(dgq):
    # full layer size: pack -> unpack is the identity, all formats, 4-bit
    codes = torch.randint(0, 16, (4096, 11008), dtype=torch.uint8, device="cuda")
    for fmt in (1, 2, 3):
        assert torch.equal(dgq.unpack(dgq.pack(codes, 4, fmt), 11008, 4, fmt), codes)


def test_bad_arguments(dgq):
    codes = torch.zeros((4, 7), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        dgq.pack(codes, 4, dgq.FMT_BYTES_HI_FIRST)   # odd column count in format 1
    with pytest.raises(RuntimeError):
        dgq.pack(codes, 5, dgq.FMT_BYTES_LO_FIRST)
    with pytest.raises(RuntimeError):
        dgq.pack(codes.cpu(), 4, dgq.FMT_BYTES_LO_FIRST)   # no CPU path

"""Hessian preparation, act-order permutation and the inverse factor against the oracle."""
import pytest
import torch

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def _spd(K, seed, Tk=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Tk or 4 * K, K, generator=g)
    idx = torch.randperm(K, generator=g)[:max(1, K // 100)]
    x[:, idx] *= 20
    x = x.bfloat16().float()
    return x.t() @ x


@pytest.mark.parametrize("K", [8, 64, 96, 200, 257, 320, 1000, 2048])
def test_inv_chol_upper(dgq, K):
    H = _spd(K, K) * (2.0 / 4)
    want = O.damped_inv_chol(H.double(), 0.01).float()      # fp64 oracle as the yardstick
    A = H.clone()
    d = torch.diagonal(A)
    d += 0.01 * d.mean()
    info = dgq.new_info("cuda")
    U = dgq.inv_chol_upper(A.cuda(), info)
    dgq.raise_on_info(info, "inv_chol")
    U = U.cpu()
    assert float(torch.tril(U, -1).abs().max()) == 0
    err = float((U - want).norm() / want.norm())
    ref32 = O.damped_inv_chol(H, 0.01)
    err32 = float((ref32 - want).norm() / want.norm())
    # as accurate as the oracle's own fp32 chain, within a small factor
    assert err <= max(10 * err32, 1e-5), (err, err32)
    # U^T U A = I
    Ad = H.double() + 0.01 * torch.diagonal(H).double().mean() * torch.eye(K, dtype=torch.float64)
    resid = (U.double().t() @ U.double() @ Ad - torch.eye(K, dtype=torch.float64)).abs().max()
    assert float(resid) < 5e-3


def test_inv_chol_matches_committed_factor(dgq, oracle_cases):
    from tests.golden.make_golden import ORACLE_CASES
    c = oracle_cases
    for name in ORACLE_CASES:
        N_out, K, Tk, bits, g, B, act, nseq = c[f"{name}_cfg"].tolist()
        H = T(c[f"{name}_H"]).cuda()
        scale = float(torch.tensor(2.0 / nseq, dtype=torch.float32))
        perm = None
        if act:
            perm, inv = dgq.actorder_perm(H, scale)
            Hs = T(c[f"{name}_H"]) * scale
            want_perm = torch.argsort(torch.diagonal(Hs), descending=True, stable=True)
            assert torch.equal(perm.cpu().long(), want_perm)
            assert torch.equal(inv.cpu().long(), torch.argsort(want_perm))
        Hp, dead = dgq.hessian_prepare(H, scale, 0.01, perm)
        assert int(dead.sum()) == 0
        U = dgq.inv_chol_upper(Hp).cpu()
        want = T(c[f"{name}_U"])
        assert float((U - want).norm() / want.norm()) < 1e-3, name


def test_not_positive_definite_is_reported(dgq):
    A = torch.eye(100, device="cuda")
    A[40, 40] = -1.0
    info = dgq.new_info("cuda")
    dgq.inv_chol_upper(A, info)
    code, idx = info.tolist()
    assert code == dgq.INFO_NOT_POSDEF and idx == 40
    with pytest.raises(RuntimeError, match="positive definite"):
        dgq.raise_on_info(info, "inv_chol")


def test_prepare_dead_columns_and_damping(dgq):
    K = 96
    H = _spd(K, 3)
    H[:, 7] = 0
    H[7, :] = 0
    H[:, 50] = 0
    H[50, :] = 0
    scale = 0.5
    Hp, dead = dgq.hessian_prepare(H.cuda(), scale, 0.01, None)
    want = H * scale
    want[7, 7] = 1
    want[50, 50] = 1
    d = torch.diagonal(want)
    d += 0.01 * d.mean()
    assert dead.cpu().nonzero().flatten().tolist() == [7, 50]
    assert torch.allclose(Hp.cpu(), want, rtol=1e-6, atol=0)
    W = torch.randn(5, K)
    Wp = dgq.permute_cols(W.cuda(), None, dead)
    W[:, [7, 50]] = 0
    assert torch.equal(Wp.cpu(), W)
    # with act-order the dead columns sort where a diagonal of 1 belongs
    perm, inv = dgq.actorder_perm(H.cuda(), scale)
    key = torch.diagonal(H * scale).clone()
    key[key == 0] = 1
    assert torch.equal(perm.cpu().long(), torch.argsort(key, descending=True, stable=True))
    codes = torch.randint(0, 16, (4, K), dtype=torch.uint8)
    assert torch.equal(dgq.permute_cols(codes.cuda(), perm).cpu(), codes[:, perm.cpu().long()])

"""Chains of independent layers on side streams: GPTQ.quantize_launch / quantize_finish and
ChainPool give exactly the results of GPTQ.quantize on the caller's stream."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


def _layers(n=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = [(256, 384), (512, 256), (128, 640), (384, 384), (256, 1024), (640, 128)][:n]
    out = []
    for i, (no, k) in enumerate(shapes):
        lin = nn.Linear(k, no, bias=False)
        lin.weight.data = torch.randn(no, k, generator=g) * 0.05
        x = torch.randn(4, 512, k, generator=g)
        x[..., ::37] *= 8.0
        out.append((lin, x))
    return out


def _run(dgq, pool, actorder):
    from distributed_gptq_b200 import GPTQ
    dev = torch.device("cuda")
    qs = []
    for lin, x in _layers():
        lin = lin.to(dev)
        q = GPTQ(lin, bits=4, group_size=128, actorder=actorder, device=dev)
        q.add_batch(x.to(dev).to(torch.bfloat16), None)
        qs.append(q)
    if pool is None:
        stats = [q.quantize() for q in qs]
    else:
        futs = [pool.submit(q.quantize_launch) for q in qs]
        for f in futs:
            f.result()
        stats = [q.quantize_finish() for q in qs]
        pool.join()
    torch.cuda.synchronize()
    return [(q.codes.cpu(), q.scale.cpu(), q.zero.cpu(), q.g_idx.cpu(),
             q.layer.weight.data.float().cpu(), s["total_error"]) for q, s in zip(qs, stats)]


@pytest.mark.parametrize("threads", [False, True])
@pytest.mark.parametrize("actorder", [False, True])
def test_chain_pool_matches_single_stream(dgq, threads, actorder):
    from distributed_gptq_b200 import ChainPool
    want = _run(dgq, None, actorder)
    pool = ChainPool(torch.device("cuda"), n_streams=3, threads=threads)
    for _ in range(2):                      # the pool is reused, as a driver does
        got = _run(dgq, pool, actorder)
        for w, g in zip(want, got):
            for a, b in zip(w[:5], g[:5]):
                assert torch.equal(a, b)
            assert abs(w[5] - g[5]) <= 1e-9 * abs(w[5])     # summed with atomics: order varies
    pool.shutdown()


def test_finish_without_launch_and_failure_restores_weight(dgq):
    from distributed_gptq_b200 import GPTQ
    dev = torch.device("cuda")
    lin = nn.Linear(128, 64, bias=False).to(dev)
    q = GPTQ(lin, bits=4, group_size=128, device=dev)
    with pytest.raises(RuntimeError):
        q.quantize_finish()
    # a Hessian that is not positive definite even after damping: the inverse reports it, the
    # layer keeps its weight and the object holds no codes
    q.H = -torch.eye(128)
    q.nsamples = 1
    before = lin.weight.data.clone()
    q.quantize_launch()
    with pytest.raises(RuntimeError, match="positive definite"):
        q.quantize_finish()
    assert torch.equal(lin.weight.data, before) and q.codes is None


def test_submit_propagates_exceptions(dgq):
    from distributed_gptq_b200 import ChainPool
    pool = ChainPool(torch.device("cuda"), n_streams=2, threads=True)

    def boom():
        raise ValueError("boom")
    fut = pool.submit(boom)
    with pytest.raises(ValueError):
        fut.result()
    with pytest.raises(ValueError):
        pool.join()
    pool.join()                              # nothing left over
    pool.shutdown()

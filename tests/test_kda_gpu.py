"""The `kda` leaf (chunkwise gated linear attention, examples/kda_fp32.ph) on a B200 against the f64
recurrence of the oracle.  The reference has no numeric check of its own for this kernel: parity is
against the recurrence its source states, with an f32 / ex2.approx tolerance written here."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL_KDA = 2e-5          # relative Frobenius: f32 accumulation over 64-token chunks, ex2.approx decay factors


def _inputs(oracle, n, d=64, gate=0.2):
    q, k, v = (oracle.lcg_fill(s, n * d).reshape(n, d) for s in (7, 8, 9))
    g = (-np.abs(oracle.lcg_fill(10, n)) * gate).astype(np.float32).reshape(n, 1)
    return q, k, v, g


@pytest.mark.parametrize("n", [64, 256, 200, 4, 1024])
def test_kda_matches_the_recurrence(ph, oracle, dev, n):
    import torch
    q, k, v, g = _inputs(oracle, n)
    Q, K, V, G = (torch.from_numpy(x).to(dev) for x in (q, k, v, g))
    O = torch.full((n, 64), float("nan"), dtype=torch.float32, device=dev)
    ph.kda(Q, K, V, G, O, 0.125)
    assert ph.device_status() == 0
    want = oracle.kda(q, k, v, g, 0.125)
    assert oracle.rel_frobenius(O.cpu().numpy(), want) <= TOL_KDA
    # by entry name, as a COMPUTE would reach it
    O.fill_(float("nan"))
    ph.launch("kda", [Q, K, V, G, O], [ph.scalar_f32(5, 0.125)])
    assert oracle.rel_frobenius(O.cpu().numpy(), want) <= TOL_KDA


def test_kda_strong_decay_and_errors(ph, oracle, dev):
    import torch
    n = 512
    # gates down to 1/e per token: the state forgets within a chunk.  (Much stronger gates overflow exp(-b) in
    # f32 inside a 64-token chunk; that is a property of the kernel's formulation, kda_fp32.ph:38-45.)
    q, k, v, g = _inputs(oracle, n, gate=1.0)
    Q, K, V, G = (torch.from_numpy(x).to(dev) for x in (q, k, v, g))
    O = torch.empty((n, 64), dtype=torch.float32, device=dev)
    ph.kda(Q, K, V, G, O, 1.0)
    assert oracle.rel_frobenius(O.cpu().numpy(), oracle.kda(q, k, v, g, 1.0)) <= 1e-4
    with pytest.raises(ph.PhobosError):
        ph.kda(Q, K, V, G[: n - 4], O, 1.0)
    with pytest.raises(ph.PhobosError):
        ph.kda(Q[:, :32].contiguous(), K[:, :32].contiguous(), V[:, :32].contiguous(), G, O[:, :32].contiguous(), 1.0)

"""Parity of the flash-attention leaves with the CPU oracle (f64 online softmax over
f16-rounded inputs, phobos-bench/src/main.rs:869-920), through the C ABI, on a B200.
Tolerance: relative Frobenius error <= 2e-3 per head."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _qkv(oracle, BH, Nq, Nk, D, normal=True, seeds=(4, 5, 6)):
    gen = oracle.lcg_fill_normal if normal else oracle.lcg_fill
    q = oracle.fp16_round(gen(seeds[0], BH * Nq * D)).reshape(BH, Nq, D)
    k = oracle.fp16_round(gen(seeds[1], BH * Nk * D)).reshape(BH, Nk, D)
    v = oracle.fp16_round(gen(seeds[2], BH * Nk * D)).reshape(BH, Nk, D)
    return q, k, v


@pytest.mark.parametrize("BH,Nq,Nk,D", [(1, 256, 128, 128), (2, 256, 384, 128), (1, 512, 1024, 64),
                                        (3, 200, 328, 128), (1, 8, 8, 64), (2, 1024, 2048, 128)])
def test_flash_fp16_matches_oracle(ph, oracle, dev, BH, Nq, Nk, D):
    import torch
    q, k, v = _qkv(oracle, BH, Nq, Nk, D)
    scale = 1.0 / np.sqrt(D)
    Q, K, V = (torch.from_numpy(x).to(dev).half() for x in (q, k, v))
    O = torch.full_like(Q, float("nan"))
    ph.flash_attention(Q, K, V, O, scale)
    assert ph.device_status() == 0
    got = O.float().cpu().numpy()
    assert np.isfinite(got).all()
    for h in range(BH):
        want = oracle.flash_rows(q[h], k[h], v[h], scale)
        assert oracle.rel_frobenius(got[h], want) <= TOL
        # the reference's sampled criterion: 2e-2 normalised by max(|want|, 0.1)  (main.rs:879, 913)
        assert oracle.max_rel_floor(got[h], want, 0.1) < 2e-2


def test_flash_reference_bench_shape(ph, oracle, dev):
    """The reference bench's own case: one head, Nq = Nk = 4096, D = 64, uniform[-1,1), scale 1/8
    (phobos-bench/src/main.rs:1062-1076); 256 sampled rows against the oracle."""
    import torch
    q, k, v = _qkv(oracle, 1, 4096, 4096, 64, normal=False)
    Q, K, V = (torch.from_numpy(x[0]).to(dev).half() for x in (q, k, v))
    O = torch.empty_like(Q)
    ph.flash_attention(Q, K, V, O, 0.125)
    assert ph.device_status() == 0
    rows = np.unique(np.concatenate([oracle.sample_points(4096, 64)[:, 0], np.arange(0, 4096, 21, dtype=np.uint64)]))
    want = oracle.flash_rows(q[0], k[0], v[0], 0.125, rows=rows)
    got = O.float().cpu().numpy()[rows.astype(int)]
    assert oracle.rel_frobenius(got, want) <= TOL


def test_flash_large_scores_need_rescale(ph, oracle, dev):
    """Scores that grow along the keys force the running maximum (and the rescale path) to move."""
    import torch
    BH, Nq, Nk, D = 1, 256, 1024, 128
    q, k, v = _qkv(oracle, BH, Nq, Nk, D)
    k = oracle.fp16_round(k * np.linspace(0.2, 6.0, Nk, dtype=np.float32)[None, :, None])
    scale = 1.0 / np.sqrt(D)
    Q, K, V = (torch.from_numpy(x).to(dev).half() for x in (q, k, v))
    O = torch.empty_like(Q)
    ph.flash_attention(Q, K, V, O, scale)
    assert ph.device_status() == 0
    want = oracle.flash_rows(q[0], k[0], v[0], scale)
    assert oracle.rel_frobenius(O.float().cpu().numpy()[0], want) <= TOL


def test_flash_negative_scale(ph, oracle, dev):
    import torch
    q, k, v = _qkv(oracle, 1, 256, 256, 64)
    Q, K, V = (torch.from_numpy(x[0]).to(dev).half() for x in (q, k, v))
    O = torch.empty_like(Q)
    ph.flash_attention(Q, K, V, O, -0.125)
    assert ph.device_status() == 0
    want = oracle.flash_rows(q[0], k[0], v[0], -0.125)
    assert oracle.rel_frobenius(O.float().cpu().numpy(), want) <= TOL


def test_flash_fp32_storage(ph, oracle, dev):
    """flash_fp32: f32 Q/K/V/O, operands rounded to f16 for the tensor cores
    (phobos-lang/src/codegen/matmul.rs:1592-1597); oracle sees the rounded inputs."""
    import torch
    BH, Nq, Nk, D = 2, 256, 512, 64
    gen = oracle.lcg_fill
    q = gen(7, BH * Nq * D).reshape(BH, Nq, D)
    k = gen(8, BH * Nk * D).reshape(BH, Nk, D)
    v = gen(9, BH * Nk * D).reshape(BH, Nk, D)
    Q, K, V = (torch.from_numpy(x).to(dev) for x in (q, k, v))
    O = torch.empty_like(Q)
    with pytest.raises(ph.PhobosError) as e:
        ph.flash_attention(Q, K, V, O, 0.125)
    assert e.value.code == ph.PH_ERR_WORKSPACE
    ws = torch.empty(ph.flash_workspace_bytes(ph.F32, BH, Nq, Nk, D), dtype=torch.uint8, device=dev)
    ph.flash_attention(Q, K, V, O, 0.125, workspace=ws)
    assert ph.device_status() == 0
    got = O.cpu().numpy()
    for h in range(BH):
        want = oracle.flash_rows(oracle.fp16_round(q[h]), oracle.fp16_round(k[h]), oracle.fp16_round(v[h]), 0.125)
        assert oracle.rel_frobenius(got[h], want) <= TOL


def test_flash_by_entry_name(ph, oracle, dev):
    """COMPUTE form: flash_attention(Q, K, V, O, scale) with the scalar at parameter position 4."""
    import torch
    q, k, v = _qkv(oracle, 1, 256, 256, 128)
    Q, K, V = (torch.from_numpy(x[0]).to(dev).half() for x in (q, k, v))
    O = torch.empty_like(Q)
    ph.launch("flash_attention", [Q, K, V, O], [ph.scalar_f32(4, 0.0883883)], grid=(2, 1, 1), cta=(128, 1, 1))
    assert ph.device_status() == 0
    want = oracle.flash_rows(q[0], k[0], v[0], 0.0883883)
    assert oracle.rel_frobenius(O.float().cpu().numpy(), want) <= TOL

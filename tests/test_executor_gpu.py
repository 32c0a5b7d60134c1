"""The instruction executor and the small device helpers, on a B200, through the C ABI."""
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_generator_matches_oracle(ph, oracle, dev):
    import torch
    n = 1_000_003
    t = torch.empty(n, device=dev)
    ph.fill_random(t, seed=1)
    assert np.array_equal(t.cpu().numpy(), oracle.lcg_fill(1, n))
    ph.fill_random(t[:4096], seed=7, first=12345, scale=0.5)
    assert np.array_equal(t[:4096].cpu().numpy(), oracle.lcg_fill(7, 12345 + 4096, 0.5)[12345:])
    h = torch.empty(8192, device=dev, dtype=torch.float16)
    ph.fill_random(h, seed=2)
    assert np.array_equal(h.float().cpu().numpy(), oracle.fp16_round(oracle.lcg_fill(2, 8192)))
    blk = torch.zeros(37, 200, device=dev)[:, :136]                       # a strided block of a 512-wide tensor
    ph.fill_random_block(blk, seed=3, first=5 * 512 + 64, stream_pitch=512)
    full = oracle.lcg_fill(3, 64 * 512).reshape(64, 512)
    assert np.array_equal(blk.cpu().numpy(), full[5:42, 64:200])
    g = torch.empty(1 << 18, device=dev)
    ph.fill_random(g, seed=4, normal=True)
    want = oracle.lcg_fill_normal(4, 1 << 18)
    assert np.allclose(g.cpu().numpy(), want, rtol=0, atol=2e-6)          # libm vs device log/sincos


def test_matmul_job_through_the_executor(ph, oracle, dev, tmp_path):
    """ALLOC, LOAD, COMPUTE(init), COMPUTE(step) x2, STORE, FREE with dependencies, for a 2x1x2 split of
    a 256x128x256 matmul read from and written to file:// tensors (cf. phobos-pod/examples/loopback.rs).
    As in a reference plan the step COMPUTEs carry the kernel's whole scalar list (alpha AND the job's
    beta = 1.5), but the step leaf is C = alpha*A@B + C: beta was applied once by the init leaf
    (phobos-cluster/src/clustergen.rs:1363-1399)."""
    M, N, K = 256, 128, 256
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    uris = [f"file://{tmp_path}/{n}.tensor" for n in "abc"]
    for uri, x in zip(uris, (a, b, c)):
        ph.store_region(uri, x.shape, (0, 0), x)
    I, tid = ph.Instr, ph.tile_id
    ins, iid = [], [0]

    def add(**kw):
        iid[0] += 1
        ins.append(I(iid=iid[0], **kw))
        return iid[0]

    with ph.Executor(0, 0, 8 << 20) as ex:
        ex.set_tensors([(uris[0], ph.F32, (M, K), ph.READ), (uris[1], ph.F32, (K, N), ph.READ), (uris[2], ph.F32, (M, N), ph.RMW)])
        ex.set_kernel(0, "matmul")
        ex.set_kernel(1, "matmul_init")
        KT, MT = K // 2, M // 2
        b_loads = []
        for kt in range(2):
            t = tid(1, 0, kt)
            al = add(op=ph.OP_ALLOC, tile=t, shape=(KT, N), data_type=ph.F32)
            b_loads.append((t, add(op=ph.OP_LOAD, tile=t, tensor=1, region_offset=(kt * KT, 0), region_shape=(KT, N), deps=(al,))))
        last = []
        for mt in range(2):
            ct = tid(2, 0, mt)
            al = add(op=ph.OP_ALLOC, tile=ct, shape=(MT, N), data_type=ph.F32)
            ld = add(op=ph.OP_LOAD, tile=ct, tensor=2, region_offset=(mt * MT, 0), region_shape=(MT, N), deps=(al,))
            prev = add(op=ph.OP_COMPUTE, kernel=1, args=((ct, ph.RMW),), scalars=(ph.scalar_f32(1, 1.5),), deps=(ld,))
            for kt in range(2):
                at = tid(0, 0, mt * 2 + kt)
                al = add(op=ph.OP_ALLOC, tile=at, shape=(MT, KT), data_type=ph.F32)
                ld = add(op=ph.OP_LOAD, tile=at, tensor=0, region_offset=(mt * MT, kt * KT), region_shape=(MT, KT), deps=(al,))
                prev = add(op=ph.OP_COMPUTE, kernel=0, args=((at, ph.READ), (b_loads[kt][0], ph.READ), (ct, ph.RMW)),
                           scalars=(ph.scalar_f32(3, 0.125), ph.scalar_f32(4, 1.5)), grid=(4, 4, 1), deps=(ld, b_loads[kt][1], prev))
                add(op=ph.OP_FREE, tile=at, deps=(prev,))
            st = add(op=ph.OP_STORE, tile=ct, tensor=2, region_offset=(mt * MT, 0), region_shape=(MT, N), deps=(prev,))
            last.append(add(op=ph.OP_FREE, tile=ct, deps=(st,)))
        for t, _ in b_loads:
            add(op=ph.OP_FREE, tile=t, deps=tuple(last))
        ex.issue(ins)
        ex.run()
        done = ex.completions()
        assert sorted(d[0] for d in done) == list(range(1, iid[0] + 1)) and all(d[1] == 0 for d in done)
        assert ex.arena_used == 0
    got = ph.load_region(uris[2], (M, N), (0, 0), (M, N))
    assert oracle.rel_frobenius(got, oracle.gemm_rows(a, b, c, 0.125, 1.5)) <= 1e-5


def test_executor_parks_allocs_until_a_free(ph, dev):
    """An ALLOC that does not fit waits for a FREE (phobos-pod/src/engine.rs:400-410, 736-742)."""
    I, tid = ph.Instr, ph.tile_id
    with ph.Executor(0, 0, 3 << 20) as ex:
        ex.issue([I(iid=1, op=ph.OP_ALLOC, tile=tid(0, 0, 0), shape=(512, 1024), data_type=ph.F32),      # 2 MiB
                  I(iid=2, op=ph.OP_ALLOC, tile=tid(0, 0, 1), shape=(512, 1024), data_type=ph.F32),      # does not fit yet
                  I(iid=3, op=ph.OP_FREE, tile=tid(0, 0, 0), deps=(1,)),
                  I(iid=4, op=ph.OP_FREE, tile=tid(0, 0, 1), deps=(2,))])
        ex.run()
        assert [d[0] for d in ex.completions()] == [1, 3, 2, 4]
        assert ex.arena_used == 0


def test_executor_reports_arena_exhaustion_and_bad_programs(ph, dev):
    I, tid = ph.Instr, ph.tile_id
    with ph.Executor(0, 0, 1 << 20) as ex:
        ex.issue([I(iid=1, op=ph.OP_ALLOC, tile=tid(0, 0, 0), shape=(1024, 1024), data_type=ph.F32)])
        with pytest.raises(ph.PhobosError) as e:
            ex.run()
        assert e.value.code == ph.PH_ERR_STATE and "arena exhausted" in e.value.message   # engine.rs:752-775
    with ph.Executor(0, 0, 1 << 20) as ex:
        ex.set_kernel(0, "conv2d")    # no such leaf
        ex.issue([I(iid=1, op=ph.OP_ALLOC, tile=tid(0, 0, 0), shape=(64, 64), data_type=ph.F32),
                  I(iid=2, op=ph.OP_COMPUTE, kernel=0, args=((tid(0, 0, 0), ph.RMW),), deps=(1,))])
        with pytest.raises(ph.PhobosError) as e:
            ex.run()
        assert e.value.code == ph.PH_ERR_UNSUPPORTED
    with ph.Executor(0, 0, 1 << 20) as ex:
        ex.issue([I(iid=1, op=ph.OP_FREE, tile=tid(5, 0, 0))])
        with pytest.raises(ph.PhobosError):
            ex.run()


def test_store_region_must_match_the_tile(ph, dev, tmp_path):
    """A STORE whose region holds more elements than the tile is refused (the reference:
    "store data/region length mismatch", phobos-cluster/src/storage.rs store_f32) and the file stays as it was."""
    I, tid = ph.Instr, ph.tile_id
    uri = f"file://{tmp_path}/c.tensor"
    ph.store_region(uri, (64, 64), (0, 0), np.ones((64, 64), dtype=np.float32))
    before = (tmp_path / "c.tensor").read_bytes()
    with ph.Executor(0, 0, 1 << 20) as ex:
        ex.set_tensors([(uri, ph.F32, (64, 64), ph.RMW)])
        ex.issue([I(iid=1, op=ph.OP_ALLOC, tile=tid(0, 0, 0), shape=(16, 16), data_type=ph.F32),
                  I(iid=2, op=ph.OP_LOAD, tile=tid(0, 0, 0), tensor=0, region_offset=(0, 0), region_shape=(16, 16), deps=(1,)),
                  I(iid=3, op=ph.OP_STORE, tile=tid(0, 0, 0), tensor=0, region_offset=(0, 0), region_shape=(32, 32), deps=(2,))])
        with pytest.raises(ph.PhobosError) as e:
            ex.run()
        assert e.value.code == ph.PH_ERR_STATE and "STORE region" in e.value.message
    assert (tmp_path / "c.tensor").read_bytes() == before


def test_f16_job_through_the_executor(ph, oracle, dev, tmp_path):
    """f16 tiles end to end (the reference's tile store sizes everything as f32, tile_store.rs:110-113)."""
    I, tid = ph.Instr, ph.tile_id
    M, N, K = 128, 256, 192
    a = oracle.fp16_round(oracle.lcg_fill(1, M * K, 0.5)).reshape(M, K)
    b = oracle.fp16_round(oracle.lcg_fill(2, K * N, 0.5)).reshape(K, N)
    c = oracle.fp16_round(oracle.lcg_fill(3, M * N, 0.5)).reshape(M, N)
    uris = [f"file://{tmp_path}/{n}.tensor" for n in "abc"]
    for uri, x in zip(uris, (a, b, c)):
        ph.store_region(uri, x.shape, (0, 0), x.astype(np.float16))
    shapes = [(M, K), (K, N), (M, N)]
    with ph.Executor(0, 0, 4 << 20) as ex:
        ex.set_tensors([(u, ph.F16, sh, md) for u, sh, md in zip(uris, shapes, (ph.READ, ph.READ, ph.RMW))])
        ex.set_kernel(0, "gemm")
        ins = []
        for t, sh in enumerate(shapes):
            ins.append(I(iid=2 * t + 1, op=ph.OP_ALLOC, tile=tid(t, 0, 0), shape=sh, data_type=ph.F16))
            ins.append(I(iid=2 * t + 2, op=ph.OP_LOAD, tile=tid(t, 0, 0), tensor=t, region_offset=(0, 0), region_shape=sh,
                         deps=(2 * t + 1,)))
        ins.append(I(iid=7, op=ph.OP_COMPUTE, kernel=0, args=((tid(0, 0, 0), ph.READ), (tid(1, 0, 0), ph.READ), (tid(2, 0, 0), ph.RMW)),
                     scalars=(ph.scalar_f32(3, 1.0), ph.scalar_f32(4, 1.0)), deps=(2, 4, 6)))
        ins.append(I(iid=8, op=ph.OP_STORE, tile=tid(2, 0, 0), tensor=2, region_offset=(0, 0), region_shape=(M, N), deps=(7,)))
        ex.issue(ins)
        ex.run()
    got = ph.load_region(uris[2], (M, N), (0, 0), (M, N), dtype=ph.F16).astype(np.float32)
    assert oracle.rel_frobenius(got, oracle.gemm_rows(a, b, c, 1.0, 1.0)) <= 1e-2


def test_fetch_of_loaded_tile(ph, oracle, dev, tmp_path):
    import torch
    I, tid = ph.Instr, ph.tile_id
    M, K = 128, 256
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    uri = f"file://{tmp_path}/a.tensor"
    ph.store_region(uri, (M, K), (0, 0), a)
    ndev = torch.cuda.device_count()
    with ph.Executor(0, 0, 4 << 20) as home, ph.Executor(1 if ndev > 1 else 0, 1, 4 << 20) as other:
        other.connect_peer(0, home)
        at = tid(0, 0, 0)
        home.set_tensors([(uri, ph.F32, (M, K), ph.READ)])
        home.issue([I(iid=1, op=ph.OP_ALLOC, tile=at, shape=(M, K), data_type=ph.F32),
                    I(iid=2, op=ph.OP_LOAD, tile=at, tensor=0, region_offset=(0, 0), region_shape=(M, K), deps=(1,)),
                    I(iid=3, op=ph.OP_FREE, tile=at, deps=(2,), expected_serves=1)])
        other.issue([I(iid=10, op=ph.OP_ALLOC, tile=at, shape=(M, K), data_type=ph.F32),
                     I(iid=11, op=ph.OP_FETCH, tile=at, from_node=0, deps=(10,))])
        import threading
        err = []

        def run_home():
            try:
                home.run()          # LOAD completes, FREE waits until the tile was served once
            except Exception as ex_:  # noqa: BLE001
                err.append(ex_)
        th = threading.Thread(target=run_home)
        th.start()
        other.run()
        th.join(timeout=60)
        assert not th.is_alive() and not err
        assert home.served_bytes == M * K * 4 and home.arena_used == 0
        addr, resident = other.tile_addr(at)
        assert resident
        # read the fetched tile back through the leaf itself: C = 1 * A @ I + 0 * C is exact in f32
        d = torch.device("cuda", 1 if ndev > 1 else 0)
        torch.cuda.set_device(d)
        eye = torch.eye(K, device=d)
        out = torch.zeros(M, K, device=d)
        A = ph.raw_desc(addr, ph.F32, M, K)
        import ctypes
        ph.check(ph.lib().phobos_gemm(ctypes.byref(A), ctypes.byref(ph.tensor_desc(eye)), ctypes.byref(ph.tensor_desc(out)),
                                      1.0, 0.0, ph.GEMM_FP32, None, 0, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        torch.cuda.set_device(0)
        assert np.array_equal(out.cpu().numpy(), a)

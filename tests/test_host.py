"""Host side of the C ABI without a GPU: the library loads and exports every declared symbol, tile ids,
size classes, the host generator, file:// storage and the job-file reader behave as the reference's."""
import json
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
G = Path(__file__).resolve().parent / "golden"


def test_library_exports_every_declared_symbol(ph):
    header = (ROOT / "include" / "phobos_leaf.h").read_text()
    declared = set(re.findall(r"\b(phobos_[a-z0-9_]+)\s*\(", header))
    assert len(declared) > 40
    out = subprocess.run(["nm", "-D", "--defined-only", str(ph.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r" T (phobos_[a-z0-9_]+)", out))
    assert declared <= exported, f"declared but not exported: {sorted(declared - exported)}"
    ph.lib()   # binds every signature
    assert b"sm_100a" in ph.lib().phobos_version()


def test_product_does_not_link_or_import_the_oracle(ph):
    out = subprocess.run(["ldd", str(ph.LIB_PATH)], capture_output=True, text=True).stdout
    assert "oracle" not in out
    for p in (ROOT / "phobos-lang_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".h"):
            text = p.read_text()
            assert "import oracle" not in text and "phobos_oracle" not in text, p


def test_tile_ids_and_size_classes(ph):
    g = json.loads((G / "tile.json").read_text())
    for t, v, c, want in g["ids"]:
        tid = ph.tile_id(t, v, c)
        assert str(tid) == want
        assert ph.tile_fields(tid) == (t, v, c)          # phobos-cluster/src/tile.rs:116-127
    for nbytes, want in g["size_class"]:
        assert ph.size_class(nbytes) == want              # phobos-pod/src/tile_store.rs:228-242
    assert [ph.lib().phobos_dtype_bytes(d) for d in range(7)] == [2, 4, 8, 1, 4, 8, 1]   # tile.rs:43-52


def test_host_generator_matches_golden_and_oracle(ph, oracle):
    g = json.loads((G / "lcg.json").read_text())
    for seed in ("1", "2", "42"):
        assert ph.fill_random_host(16, int(seed)).view(np.uint32).tolist() == g[seed]["unit_bits"]
    sk = g["skip"]
    assert int(ph.fill_random_host(1, sk["seed"], first=sk["index"]).view(np.uint32)[0]) == sk["unit_bits"]
    assert np.array_equal(ph.fill_random_host(1000, 9, first=123, scale=0.5), oracle.lcg_fill(9, 1123, 0.5)[123:])


def test_storage_region_load_store(ph, tmp_path):
    """Row-span gather / scatter without truncation (phobos-cluster/src/storage.rs:22-79)."""
    uri = f"file://{tmp_path}/t.tensor"
    full = np.arange(12 * 10, dtype=np.float32).reshape(12, 10)
    ph.store_region(uri, (12, 10), (0, 0), full)
    assert (tmp_path / "t.tensor").stat().st_size == 12 * 10 * 4
    tile = ph.load_region(uri, (12, 10), (3, 4), (5, 6))
    assert np.array_equal(tile, full[3:8, 4:10])
    ph.store_region(uri, (12, 10), (2, 1), np.full((2, 3), -1.0, dtype=np.float32))
    back = ph.load_region(uri, (12, 10), (0, 0), (12, 10))
    want = full.copy()
    want[2:4, 1:4] = -1.0
    assert np.array_equal(back, want)
    assert np.array_equal(ph.load_region(uri, (120,), (7,), (5,)), want.ravel()[7:12])   # rank 1
    h = np.arange(32, dtype=np.float16).reshape(4, 8)                                     # f16 tiles
    ph.store_region(f"file://{tmp_path}/h.tensor", (4, 8), (0, 0), h)
    assert np.array_equal(ph.load_region(f"file://{tmp_path}/h.tensor", (4, 8), (1, 2), (2, 4), dtype=ph.F16), h[1:3, 2:6])
    assert ph.storage_path("file:///C:/x/a.tensor") == "C:/x/a.tensor"                    # storage.rs:14-18
    with pytest.raises(ph.PhobosError) as e:
        ph.storage_path("s3://bucket/x")
    assert "expected file://" in e.value.message
    with pytest.raises(ph.PhobosError) as e:
        ph.load_region(f"file://{tmp_path}/missing", (4, 4), (0, 0), (2, 2))
    assert e.value.code == ph.PH_ERR_IO
    # a region wider than the tensor would wrap into the next row; one past the last row would read
    # beyond the file: both are refused before any byte moves
    before = (tmp_path / "t.tensor").read_bytes()
    for off, shape in (((0, 6), (2, 6)), ((11, 0), (2, 4)), ((0, 11), (1, 1)), ((13, 0), (1, 1))):
        with pytest.raises(ph.PhobosError) as e:
            ph.load_region(uri, (12, 10), off, shape)
        assert e.value.code == ph.PH_ERR_INVALID and "exceeds" in e.value.message
        with pytest.raises(ph.PhobosError) as e:
            ph.store_region(uri, (12, 10), off, np.zeros(shape, dtype=np.float32))
        assert e.value.code == ph.PH_ERR_INVALID
    with pytest.raises(ph.PhobosError):
        ph.load_region(uri, (120,), (118,), (5,))
    assert (tmp_path / "t.tensor").read_bytes() == before


JOB = """\
# partitioned matmul
source = {src}
dim M = 16384
dim N = 16384
dim K = 16384
tensor A = read  f32 16384x16384 file:///data/a.tensor
tensor B = read  f32 16384x16384 file:///data/b.tensor
tensor C = rmw   f32 16384x16384 file:///data/c.tensor   # in place
scalar alpha = f32 0.125
scalar beta = f32 1.5
"""
SRC = """\
@cluster(TILE_M in [4096, 16384], TILE_N in [4096, 16384], TILE_K in [4096, 16384])
// kernel comment
kernel matmul(A: tensor<f32>[M, K], B: tensor<f32>[K, N], C: tensor<f32>[M, N], alpha: f32, beta: f32) {
}
"""


def test_job_file_grammar(ph, tmp_path):
    """phobos-sched/src/job.rs:5-88 and examples/matmul_cluster_job.txt."""
    (tmp_path / "k.ph").write_text(SRC)
    (tmp_path / "job.txt").write_text(JOB.format(src=tmp_path / "k.ph"))
    job = ph.parse_job(str(tmp_path / "job.txt"))
    assert job.kernel == "matmul"
    assert job.dims == {"M": 16384, "N": 16384, "K": 16384}
    assert [(t.name, t.mode, t.dtype, t.shape) for t in job.tensors] == [
        ("A", ph.READ, ph.F32, (16384, 16384)), ("B", ph.READ, ph.F32, (16384, 16384)), ("C", ph.RMW, ph.F32, (16384, 16384))]
    assert job.tensors[2].uri == "file:///data/c.tensor"
    assert [(s.name, s.value) for s in job.scalars] == [("alpha", 0.125), ("beta", 1.5)]


@pytest.mark.parametrize("text,msg", [
    ("dim M = x\nsource = s", "dim value must be an integer"),
    ("source = s\ntensor A = rd f32 4x4 file:///a", "unknown tensor mode 'rd' (read|write|rmw)"),
    ("source = s\ntensor A = read f33 4x4 file:///a", "unknown data type 'f33'"),
    ("source = s\ntensor A = read f32 4xN file:///a", "bad shape extent 'N'"),
    ("source = s\ntensor A = read f32 4x4", "tensor missing uri"),
    ("source = s\nscalar a = f32 abc", "scalar value 'abc' is not a valid f32"),
    ("source = s\nscalar a = q8 1", "unknown scalar data type 'q8'"),
    ("source = s\nfoo bar", "unknown directive 'foo bar'"),
    ("dim M = 4", "job-file has no `source =` line"),
])
def test_job_file_errors(ph, text, msg):
    with pytest.raises(ph.PhobosError) as e:
        ph.parse_job_text(text, "job.txt", source_text="kernel k() {}")
    assert e.value.code == ph.PH_ERR_PARSE and msg in e.value.message
    if "no `source" not in msg:
        assert re.match(r"\[-7\] job.txt:\d+: ", str(e.value))


def test_job_scalars_and_types(ph):
    job = ph.parse_job_text("source = s\nscalar a = i32 -7\nscalar b = i64 1234567890123\nscalar c = bool true\n"
                            "scalar d = f64 2.5\ntensor T = write f16 128 file:///t  # rank 1\n", source_text="kernel add() {}")
    assert [s.value for s in job.scalars] == [-7, 1234567890123, True, 2.5]
    assert job.tensors[0].shape == (128,) and job.tensors[0].dtype == ph.F16 and job.tensors[0].mode == ph.WRITE
    assert job.kernel == "add"


def test_compute_calls_fail_loudly_without_a_device(ph):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    info = ph.PhDeviceInfo()
    assert ph.lib().phobos_device_info(0, info) == ph.PH_ERR_DEVICE
    with pytest.raises(ph.PhobosError):
        ph.Executor(0, 0, 1 << 20)

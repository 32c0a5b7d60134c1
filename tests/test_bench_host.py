"""Host-side pieces of bench.py that need no GPU: the reference arm and the CSV writer."""
import importlib.util
import json
import subprocess
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("phobos_bench_main", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_csv_has_the_reference_columns_and_labels(tmp_path):
    bench = load_bench()
    res = {
        "gemm_fp32": {"tflops": 52.0, "ms_per_launch": 2.64, "roofline": {"bound": "fp32_ffma", "frac": 0.70},
                      "cpu_baseline": {"value": 0.5, "kind": "port"}},
        "gemm_fp16": {"tflops": 1500.0, "ms_per_launch": 0.73, "roofline": {"bound": "tensor", "frac": 0.92}},
        "flash_fp16": {"tflops": 1100.0, "ms_per_launch": 1.0, "roofline": {"bound": "tensor", "frac": 0.67}},
    }
    args = types.SimpleNamespace(peak_fp32=None, peak_fp16tc=2000.0, peak_fp16tcf32acc=None)
    info = types.SimpleNamespace(fp32_peak_flops=74.4e12)
    out = tmp_path / "r.csv"
    bench.write_csv(out, res, args, info)
    lines = out.read_text().splitlines()
    # the reference's six columns come first, in its order (phobos-bench/src/report.rs:71-88)
    assert lines[0].startswith("benchmark,impl,precision,gflops,peak_gflops,pct_of_peak")
    rows = {(r.split(",")[0], r.split(",")[1]): r.split(",") for r in lines[1:]}
    assert rows[("gemm_fp32", "phobos-b200")][2:6] == ["f32", "52000.0", "74400.0", "69.9"]
    assert rows[("gemm_fp16", "phobos-b200")][2:6] == ["f16-tc", "1500000.0", "2000000.0", "75.0"]     # override
    assert rows[("flash_fp16", "phobos-b200")][2:6] == ["f16-tc-f32-acc", "1100000.0", "2250000.0", "48.9"]
    assert rows[("gemm_fp32", "cpu-port")][3] == "500.0"


def test_reference_arm_prints_one_json_line():
    """`--impl reference` runs the CPU restatement on a bounded sample and needs no GPU."""
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["config"]["workload"] == "gemm_fp16tc_fp32acc"
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0


def test_traffic_provenance_hashes_code_not_wording():
    """The figure of an ncu capture stays attached to a kernel while only its comments change, and is
    reported stale as soon as the code does."""
    bench = load_bench()
    a = '// header\n__global__ void k(int* p) { /* note */ p[0] = 1;  // "x"\n  const char* s = "a // b";\n}\n'
    b = '// another header, reworded\n__global__ void k(int* p) {\n  p[0] = 1;\n  const char* s = "a // b";\n}\n'
    c = a.replace("p[0] = 1", "p[0] = 2")
    d = a.replace('"a // b"', '"a / b"')
    assert bench._code_only(a) == bench._code_only(b)
    assert bench._code_only(a) != bench._code_only(c)
    assert bench._code_only(a) != bench._code_only(d)      # string literals are code
    # every entry of the committed table names a kernel source that exists and a profile that exists
    table = json.loads((ROOT / "profiles" / "ncu_traffic.json").read_text())
    for name, e in table.items():
        assert name in bench.KERNEL_FILES
        assert (ROOT / e["profile"]).exists()
        assert e["kernel_sha"] == bench.kernel_sha(name), f"{name}: the capture is older than the kernel source"

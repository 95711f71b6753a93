"""Host-side checks of bench.py that need no GPU: the CPU arm prints the contract's JSON line, and the
roofline helpers are consistent."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_the_contract_line():
    env = dict(os.environ, QUARTET_BENCH_CPU_TOKENS="128")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    b = _bench_module()
    assert line["impl"] == "reference" and line["metric"] == b.METRIC and line["unit"] == "TFLOP/s"
    assert line["config"] == b.bench_config(b.WORKLOAD, 1, "auto") and line["higher_is_better"] is True
    assert line["steps"] == 1 and line["warmup"] == 0
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True,
                       text=True, cwd=ROOT, env=env, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_flop_and_traffic_helpers(tmp_path):
    b = _bench_module()
    m = b.TOKENS
    assert b.layer_flops(m) == sum(6.0 * m * k * n for _, k, n in b.LAYERS)
    # operands at 4.25 bits per element plus the result
    assert b.gemm_algorithmic_bytes(256, 512, 1024, 2) == (256 + 512) * 1024 * (0.5 + 1 / 32) + 256 * 512 * 2
    # DRAM traffic comes from a tracked ncu summary, scaled by algorithmic bytes; without one it is None
    traffic, algorithmic = b.gemm_traffic_per_launch(b.LAYERS, m, {})
    assert traffic is None and algorithmic > 0
    md = tmp_path / "gemm.md"
    md.write_text("ncu ... python -m x --kernel gemm --m 8192 --n 8192 --k 4096\n\n| metric | unit | launch 1 | launch 2 |\n|---|---|---|---|\n"
                  "| dram__bytes_read.sum | Mbyte | 36.0 | 36.1 |\n| dram__bytes_write.sum | Mbyte | 84.0 | 83.9 |\n"
                  "| sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active | % | 66.1 | 66.0 |\n")
    cap = b.read_ncu_summary(str(md))
    assert cap["shape"] == (8192, 8192, 4096) and cap["dram__bytes_read.sum"] == 36.0e6
    traffic, algorithmic = b.gemm_traffic_per_launch(b.LAYERS, m, cap)
    ratio = 120.0e6 / b.gemm_algorithmic_bytes(8192, 8192, 4096, 2)
    assert abs(traffic / algorithmic - ratio) < 1e-12
    assert b.read_ncu_summary(str(tmp_path / "missing.md")) == {}


def test_both_arms_describe_the_same_config():
    b = _bench_module()
    assert b.bench_config(b.WORKLOAD, 1, "auto") == b.bench_config(b.WORKLOAD, 1, "copy")
    c = b.bench_config(b.WORKLOAD, 8, "auto")
    assert c["workload"] == b.WORKLOAD and c["tokens_per_gpu"] == b.TOKENS and "dp8" in c["parallelism"]
    assert b.load_peaks()["bf16_burst"] >= b.load_peaks()["bf16_sustained"] > 0

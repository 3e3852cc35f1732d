"""Host-side checks of bench.py that need no GPU: the reference arm runs on the CPU oracle without loading the CUDA
library and prints the agreed JSON line; the tracked traffic file covers the default workload; the helpers that size
the CPU sample and count window pairs."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_reference_arm_prints_the_line_and_never_loads_the_package():
    code = ("import sys, runpy; sys.argv = ['bench.py', '--impl', 'reference', '--workload', 'cfg1', '--steps', '1', "
            "'--warmup', '1']\n"
            "try:\n    runpy.run_path('bench.py', run_name='__main__')\nexcept SystemExit as e:\n    assert not e.code\n"
            "assert 'dl_templates_b200' not in sys.modules, 'the reference arm imported the product package'\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_traffic_file_covers_the_default_workload():
    import bench
    tr = bench.load_traffic()
    for k in ("fwd", "dq", "dkdv"):
        e = tr[f"target:handoff:{k}"]
        assert e["bytes_per_bh"] > 1e6 and "commit" in e["source"]


def test_cpu_sample_sizes_and_pair_count():
    import bench
    assert bench.exact_pairs(3, 1) == 49                         # (2 + 3 + 2) ** 2
    assert bench.exact_pairs(16, 3) == sum(min(15, i + 3) - max(0, i - 3) + 1 for i in range(16)) ** 2
    small, big = bench.workload_dims("target"), bench.workload_dims("cfg5")
    assert bench.cpu_band_rows(small) == 128                     # 16384 tokens: the whole grid
    assert bench.cpu_band_rows(big) == 64 and bench.cpu_slices_for(big) == 1
    assert "band of 64 full rows" in bench.cpu_sample_text(big, 1, "cfg5")

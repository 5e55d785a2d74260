"""The one JSON line bench.py prints: the keys and meanings the benchmark contract fixes.

Without a GPU: the reference arm (the reference algorithm on the host cores) on a small shape.  With a GPU: the library's own
line on a small shape, with its roofline, CPU-baseline, host-memory and clock records."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env=None):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, **(env or {})))
    assert res.returncode == 0, res.stderr[-3000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, res.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run(["--impl", "reference", "--B", "2", "--T", "128", "--H", "2", "--steps", "2", "--warmup", "1"])
    assert d["impl"] == "reference" and d["metric"] == "wkv6_fwd_bwd_mtokens_per_s" and d["unit"] == "Mtokens/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1
    assert d["value"] > 0 and abs(d["value"] - 2 * 128 / (d["ms_per_step"] * 1e-3) / 1e6) <= 1e-6 * d["value"] + 1e-12
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "sample" in cb
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"].startswith("wkv6 fwd+bwd B2 T128 H2 N64")


def test_reference_arm_other_ranks_exit_quietly():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29591"))
    assert res.returncode == 0 and not [ln for ln in res.stdout.splitlines() if ln.startswith("{")]


@pytest.mark.gpu
def test_library_line_on_a_small_shape():
    d = _run(["--B", "2", "--T", "1024", "--H", "8", "--steps", "5", "--warmup", "3", "--no-reference-cuda"])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "clocks", "gpu_launches"):
        assert key in d, key
    assert d["dtype"] == "bf16" and d["data"] == "synthetic" and d["vs_baseline"] is None and d["gpu_launches"] > 0
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] >= 5 * 2 * 1024 * 8 * 64 * 2 and e["d2h_bytes_per_step"] >= 5 * 2 * 1024 * 8 * 64 * 2
    assert 0 < e["value"] < d["value"]
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    assert d["device_status"] == 0

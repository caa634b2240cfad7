"""bench.py without a GPU: the reference arm prints the contract's JSON line with the same `config`
object as the CUDA arm would, and the DRAM-traffic record under profiles/ was captured from the
kernel sources as they are now."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _reference_line(*extra):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", *extra], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


@pytest.mark.parametrize("workload,metric,scaling", [
    ("c3", "sampled_rows_per_s_topp_v128256_bf16", "weak"),
    ("c5", "sampled_rows_per_s_topp_v256000_bf16", "strong"),
])
def test_reference_arm_line(workload, metric, scaling):
    import bench
    d = _reference_line("--workload", workload)
    assert d["impl"] == "reference" and d["metric"] == metric and d["unit"] == "rows/s"
    assert d["scaling"] == scaling and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["value"] > 0 and d["steps"] == 1 and d["gpu_launches"] == 0
    assert d["e2e"] == {"value": d["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert set(cb["variants"]) == {"float_upcast_all_threads", "native_one_thread", "float_upcast_one_thread"}
    # both arms describe the workload with the same object
    assert d["config"] == bench.config_dict(1, False, "p2p", workload)


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120,
                         cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_traffic_record_matches_kernel_sources():
    import bench
    with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
        t = json.load(f)
    assert t["source_hash"] == bench.kernel_source_hash(), \
        "kernel sources changed after the ncu capture in profiles/traffic.json: capture again"
    for name in ("sample_rows_kernel", "argmax_rows_kernel"):
        traffic, stale = bench.dram_traffic(name)
        assert not stale and 65_673_216 * 0.99 < traffic < 65_673_216 * 1.2

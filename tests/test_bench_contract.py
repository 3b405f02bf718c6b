"""Host-side pieces of the benchmark contract that need no GPU: the byte accounting behind the roofline
object, the workload labels, the recorded traffic figures, and the line the CPU arm prints."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_algorithmic_bytes_of_the_headline_workload():
    import bench
    ab = bench.algorithmic_bytes(bench.CONTEXT)
    # far pool: pages between the sink page and the near pool, 128 B of min/max rows each (d' = 32);
    # near pool: 256 pages, 64 B of sums each; 8 KV heads
    assert ab["l1"] == 8 * (7927 * 128 + 256 * 64)
    assert ab["l2"] == 8 * 130 * 16 * 20
    assert ab["attn"] == 8 * 1024 * 512 + 8 * 1024 * 4
    assert ab["total"] == ab["l1"] + ab["l2"] + ab["attn"] + ab["append"] + 2 * 32 * 128 * 2
    assert 12.8e6 < ab["total"] < 12.9e6


def test_workload_labels_name_the_partition():
    import bench
    one = bench.workload_config(1, "kvhead")
    assert one["workload"] == "cfg2-qwen3-8b-128k" and one["context"] == 131072 and one["batch"] == 1
    assert "model" not in one
    assert "KV heads" in bench.workload_config(8, "kvhead")["sharding"]
    assert "independent" in bench.workload_config(2, "request")["sharding"]


def test_recorded_traffic_is_close_to_the_algorithmic_bytes():
    import bench
    t = bench.measured_traffic("decode_step", "cfg2-qwen3-8b-128k")
    assert t is not None and 1.0 <= t / bench.algorithmic_bytes(bench.CONTEXT)["total"] < 1.1
    assert bench.measured_traffic("decode_step", "no-such-workload") is None


def test_cpu_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--skip-reference-code"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["config"]["workload"] == "cfg2-qwen3-8b-128k"
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}

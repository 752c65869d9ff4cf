"""Host-side pieces of bench.py that need no GPU: the algorithmic byte counts, the reference arm's
line, and the rule that a DRAM-traffic capture is quoted only for the kernel sources it came from."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_algorithmic_bytes_of_the_headline_workload():
    import bench
    from fstattention_b200 import configs
    w = configs.workload("medusa256")
    info = bench.describe(w)
    # 97 ancestor rows + 243 leaf rows over the four blocks, 32 heads, 128 columns, fp16, K and V
    assert info["gathered_rows_per_head"] == 97 + 243
    assert info["gathered_kv_bytes_per_call"] == 5570560
    assert info["q_o_bytes_per_call"] == 2 * 32 * 256 * 128 * 2
    cfg = bench.workload_config(w, 64)
    assert cfg["workload"] == "medusa256" and cfg["calls_per_step"] == 64 and "kernel" not in cfg


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "binary31",
                          "--steps", "3", "--warmup", "1", "--layers", "4"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "tree_attn_gathered_kv_bandwidth"
    assert line["config"]["calls_per_step"] == 4 and line["gpu_launches"] == 0
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("port", "reference") and cpu["cores"] >= 1 and cpu["value"] == line["value"]
    assert set(cpu["legs"]) == {"precompute", "attention"}
    # the step is composed from the two legs: 1 precompute + calls_per_step attention calls
    want = cpu["legs"]["precompute"]["ms_per_tree"] + 4 * cpu["legs"]["attention"]["ms_per_call_per_tree"]
    assert abs(line["ms_per_step"] - want) <= 1e-6 * max(want, 1.0)


def test_traffic_capture_is_quoted_only_for_its_sources(tmp_path, monkeypatch):
    import bench
    rec = {"kernel_sources_sha1": bench.kernel_source_digest(),
           "captures": {"medusa256": {"kernel": "k", "dram_bytes_per_launch": 123.0}}}
    path = tmp_path / "t.json"
    path.write_text(json.dumps(rec))
    monkeypatch.setattr(bench, "TRAFFIC_JSON", str(path))
    assert bench.ncu_traffic("medusa256")[0] == 123.0
    assert bench.ncu_traffic("forest64")[0] is None
    rec["kernel_sources_sha1"] = "0" * 16
    path.write_text(json.dumps(rec))
    value, why = bench.ncu_traffic("medusa256")
    assert value is None and "older" in why

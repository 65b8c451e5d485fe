"""The benchmark's reference arm (the CPU path) needs no GPU: run it on the smallest workload and check the
record it prints against the contract (same metric, unit and workload description as the GPU arm; the keys
the driver reads)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg1",
                          "--steps", "1", "--warmup", "0"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["metric"] == "edge_gflops" and rec["unit"] == "GFLOP/s"
    assert rec["higher_is_better"] is True and rec["n_gpus"] == 1 and rec["steps"] == 1 and rec["warmup"] == 0
    assert rec["value"] > 0 and rec["ms_per_step"] > 0 and rec["gpu_launches"] == 0
    assert rec["config"]["workload"].startswith("cfg1_er4096") and "model" not in rec["config"]
    cb = rec["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == rec["value"] and cb["sample"]
    e2e = rec["e2e"]
    assert e2e["value"] == rec["value"] and e2e["unit"] == rec["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert rec["full_workload_per_step"] is True  # 36 864 edges fit any budget: a measured full call


def test_both_arms_describe_the_workload_identically(monkeypatch):
    """The driver compares the two arms' ``config`` entries: they come from one function of the arguments."""
    sys.path.insert(0, ROOT)
    import bench
    from fused3s_b200 import graphs

    g = graphs.make_config(1)
    configs = []
    for impl, gpus in (("ours", "1"), ("reference", "1"), ("ours", "8"), ("reference", "8")):
        monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", impl, "--workload", "cfg1", "--gpus", gpus])
        configs.append(bench.workload_config(bench.parse_args(), g))
    assert configs[0] == configs[1] and configs[2] == configs[3]
    assert configs[0]["sharding"] == "single GPU" and configs[2]["sharding"] != "single GPU"
    assert "L2 flushed" in configs[0]["l2"] and "larger than L2" not in configs[0]["l2"]  # 36 864 edges

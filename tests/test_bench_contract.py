"""The bench line's contract, checked where no GPU is needed: the reference arm runs the CPU port on
the host cores and must print one JSON line with the keys the driver reads."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "C1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["higher_is_better"] is True
    assert line["unit"] == "tokens/s" and line["value"] > 0 and line["data"] == "synthetic"
    assert line["vs_baseline"] is None
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and line["config"]["global_batch"] == 1 and line["config"]["n_shards"] == 1
    assert line["steps"] == 1 and line["warmup"] == 0 and line["scaling"] == "strong"


def test_both_arms_name_the_job_the_same_way():
    sys.path.insert(0, ROOT)
    import bench
    for n in (1, 2, 8):
        cfg = bench.job_config("C2", bench.WORKLOADS["C2"], n)
        assert cfg["global_batch"] == 8 and cfg["n_shards"] == n          # the same job at every N: strong scaling
    sh = [bench.Shard(bench.WORKLOADS["C2"], r, 8) for r in range(8)]
    assert [s.b for s in sh] == [1] * 8 and sh[3].b_lo == 3
    sh = [bench.Shard(bench.WORKLOADS["C4"], r, 4) for r in range(4)]
    assert [s.h_k for s in sh] == [8] * 4 and sh[0].b == 32
    sh = [bench.Shard(bench.WORKLOADS["C5b"], r, 8) for r in range(8)]
    assert [s.s for s in sh] == [131072] * 8 and sh[7].t_hi == 1048576


def test_workload_table_matches_the_baseline_configs():
    sys.path.insert(0, ROOT)
    import bench
    w = bench.WORKLOADS
    assert w["C2"]["b"] == 8 and w["C2"]["h"] == 32 and w["C2"]["h_k"] == 8 and w["C2"]["s"] == 32768
    assert w["C2"]["bits"] == 4 and w["C2"]["group"] == 128 and w["C2"]["res"] == 64
    assert w["C3"]["bits"] == 2 and w["C3"]["group"] == 64 and w["C3"]["s"] == 131072
    assert w["C4"]["ragged"] and w["C4"]["dtype"] == "bf16" and w["C4"]["h"] == w["C4"]["h_k"] == 32
    # algorithmic bytes of C2: codes + scales/zeros + tail + q/out (the roofline numerator)
    assert bench.algorithmic_bytes(w["C2"]) == 287440896

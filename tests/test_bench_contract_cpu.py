"""The benchmark's reference arm runs without a GPU: its JSON line must carry the keys the contract names, and
under a multi-rank launch only rank 0 may work and print."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"}


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return [l for l in r.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_prints_one_contract_line():
    lines = _run({})
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert KEYS <= set(d) and d["impl"] == "reference"
    assert d["value"] > 0 and d["unit"] == "queries/s" and d["higher_is_better"] is True
    assert d["config"]["workload"] == "flat-euclidean-100k-d128-q1000-k10"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_other_ranks_exit_without_work():
    assert _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == []


def test_the_default_run_s_other_configurations_exist_and_cannot_recurse():
    """The default one-GPU run records further configurations as child processes: each must be a workload of the
    bench, none the default one, and a child must be told not to start children of its own."""
    sys.path.insert(0, ROOT)
    import importlib
    bench = importlib.import_module("bench")
    names = [w for w, _ in bench.OTHER_WORKLOADS]
    assert names and all(w in bench.WORKLOADS for w in names) and "c2" not in names
    assert all(steps >= 3 for _, steps in bench.OTHER_WORKLOADS)
    src = open(os.path.join(ROOT, "bench.py")).read()
    body = src[src.index("def run_other_workloads"):src.index("def main()")]
    assert '"--no-others"' in body and "timeout=" in body and "except Exception" in body

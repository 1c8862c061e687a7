"""bench.py's pure helpers on the CPU: the algorithmic byte / flop counts, the traffic figures read from the
kept ncu summary, the workload strings shared by both arms, and the argument parser's defaults."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_algorithmic_counts_are_positive_and_consistent():
    by, fl = bench.alg_bytes(bench.CFG), bench.alg_flops(bench.CFG)
    assert set(by) == set(fl) == {"prepass_fwd", "state_fwd", "state_bwd", "prepass_bwd"}
    assert all(v > 0 for v in by.values()) and all(v > 0 for v in fl.values())
    st = bench.step_alg(bench.CFG)
    # user-visible bytes of a step: inputs, output cotangent and the six gradients, each once
    c = bench.CFG
    tok = c["B"] * c["L"]
    qk = 2 * tok * c["Hk"] * c["K"] * 2
    assert st["bytes"] > qk and st["flops"] > 0


def test_traffic_line_of_the_kept_profile_parses():
    t = bench.ncu_traffic()
    assert set(t) == {"prepass_fwd", "state_fwd", "state_bwd", "prepass_bwd"}
    assert all(1e6 < v < 1e10 for v in t.values())


def test_reference_arm_names_the_same_workload():
    # the reference arm prints the main arm's metric and workload strings
    src = (ROOT / "bench.py").read_text()
    assert src.count("METRIC") >= 3 and src.count("WORKLOAD") >= 3
    assert "tokens/s" in bench.METRIC and "L=2048" in bench.WORKLOAD and "Hv=24" in bench.WORKLOAD


def test_help_lists_the_contract_flags():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in out.stdout


def test_reference_arm_prints_the_contract_line():
    """`--impl reference` needs no GPU: it times the CPU oracle on the whole workload and prints one JSON line."""
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["metric"] == bench.METRIC and line["config"]["workload"] == bench.WORKLOAD
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == dict(value=line["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)

"""`bench.py --impl reference` on the CPU: one JSON line with the contract's keys, from the reference's own einops
code when it has been placed under oracle/_ref, else from the oracle's restatement."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"] + extra
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, r.stdout
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line():
    line = _run(["--ref-tokens", "64", "--cpu-tokens", "64", "--ref-heads", "1"])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["unit"] == "Mtokens/s"
    assert line["value"] > 0 and line["ms_per_step"] > 0
    have_ref = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "fastattention_einops.py"))
    assert line["cpu_baseline"]["kind"] == ("reference" if have_ref else "port")
    assert line["cpu_baseline"]["cores"] >= 1 and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["config"]["workload"].startswith("cfg2_")


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""

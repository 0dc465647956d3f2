"""CPU test of bench.py's output contract on the arm that needs no GPU (`--impl reference`): exactly one
JSON line on stdout with the keys the driver reads, also when launched with torchrun's environment."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REQUIRED = ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
            "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e")


def _run(extra_env):
    env = dict(os.environ, **extra_env)
    # one step of the one-head N=4096 sample takes a couple of seconds on 8 cores
    res = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    return res.stdout


def test_reference_arm_prints_one_json_line():
    out = _run({})
    lines = [l for l in out.splitlines() if l.strip()]
    assert len(lines) == 1, out
    j = json.loads(lines[0])
    for k in REQUIRED:
        assert k in j, k
    assert j["impl"] == "reference" and j["unit"] == "TFLOP/s" and j["vs_baseline"] is None
    # the reference's own module when baseline/_ref holds it (installed where the reference checkout is present), else the port
    from baseline import ref_loader
    have_ref = ref_loader.installed() or os.path.isdir(os.path.join(ref_loader.default_checkout(), "src"))
    assert j["cpu_baseline"]["kind"] == ("reference" if have_ref else "port") and j["cpu_baseline"]["cores"] >= 1
    c1 = j["cpu_baseline"]["c1"]
    assert c1["shape"].startswith("B=2 H=16 N=512 D=32") and c1["timed"] >= 7 and c1["fwd_bwd_ms"] > c1["fwd_ms"] > 0
    assert j["e2e"]["h2d_bytes_per_step"] == 0 and j["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in j["config"] and "model" not in j["config"]


def test_reference_arm_other_ranks_print_nothing():
    out = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert out.strip() == ""

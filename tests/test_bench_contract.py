"""The benchmark's reference arm (the CPU restatement timed on the host cores) at a small size: it must print one
JSON line with the keys the contract names, on the workload the GPU arm uses, and stay consistent with the checker."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_the_contract_line(oracle):
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--n", "1024", "--steps", "2",
                          "--warmup", "1"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "cpu_baseline", "impl"):
        assert key in d, key
    assert d["impl"] == "reference" and d["steps"] == 2 and d["n_gpus"] == 1
    assert d["metric"] == "spamm_executed_tflops" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["value"] == d["value"] == d["cpu_baseline"]["value"]
    # the value is 65536 * S / time with S from the checker on the same seeded matrices
    from cuspamm_b200 import gen_signed_exp

    A = gen_signed_exp(0.1, 1, 1024, 1024)
    B = gen_signed_exp(0.1, 2, 1024, 1024)
    _, S = oracle.spamm(A, B, 1e-6)
    assert d["config"]["survivors"] == S
    assert abs(d["value"] - 65536.0 * S / (d["ms_per_step"] * 1e-3) / 1e12) <= 1e-9 * max(1.0, d["value"])

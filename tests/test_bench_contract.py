"""CPU-only checks of bench.py: the entry accounting and the reference arm's JSON line (tiny sample)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_entries_per_step_accounting():
    sys.path.insert(0, ROOT)
    import bench
    n = m = 50000
    # cross term: 102 Jacobi steps x 2 soft-mins + grad_x; self terms: ONE soft-min per step (f == g);
    # OT(x,x) contributes both gradient sides, OT(y,y) none
    assert bench.entries_per_step(n, m, 100, debias=True) == 204 * n * m + n * m + 102 * n * n + 2 * n * n + 102 * m * m
    assert bench.entries_per_step(n, m, 100, debias=False) == 204 * n * m + n * m
    assert bench.entries_per_step(n, m, 100, debias=True) == 1027500000000


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--n", "1500", "--d", "8"], capture_output=True, text=True, timeout=300,
                         cwd=ROOT)
    assert out.returncode == 0, out.stderr[-500:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["metric"] == "cost_entries_per_sec" and rec["unit"] == "entries/s"
    assert rec["value"] > 0 and rec["higher_is_better"] is True and rec["cpu_baseline"]["kind"] == "port"
    assert rec["cpu_baseline"]["cores"] >= 1 and rec["e2e"]["h2d_bytes_per_step"] == 0

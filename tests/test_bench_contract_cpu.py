"""CPU: the benchmark's CPU arm and JSON contract on a tiny workload (no GPU involved)."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_cpu_sample_has_the_workloads_composition():
    """The CPU arm times a sample with the same Muon / AdamW mix as the whole workload, so its
    params/s is measured on the sample and only ms_per_step of the full step is derived."""
    import bench
    from ancora_cutile_b200 import shapes as S
    shp = S.qwen3_0_6b_shapes(n_layers=3, hidden=128, q_heads=2, kv_heads=1, head_dim=128, ffn=384, vocab=2048)
    mu = bench.route(shp)
    assert len(mu) == 21
    total = S.count(shp)
    cb = bench.cpu_arm(shp, mu, total, steps=1, warmup=0, layers=1)
    assert cb["extrapolated"] and abs(cb["sample_fraction"] - 1 / 3) < 1e-9          # 1 of 3 identical layers
    m_total = sum(int(np.prod(shp[n])) for n in mu)
    a_total = total - m_total
    assert abs(cb["sample_params"] - (m_total // 3 + a_total / 3)) <= 64            # AdamW share rounded to 64
    assert cb["kind"] in ("reference", "port") and cb["value"] > 0 and cb["muon_ms"] > 0 and cb["adamw_ms"] > 0
    assert abs(cb["ms_per_step"] - total / cb["value"] * 1e3) < 1e-6
    whole = bench.cpu_arm(shp, mu, total, steps=1, warmup=0, layers=3)
    assert not whole["extrapolated"] and whole["sample_fraction"] == 1.0


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    env = dict(os.environ, ANCORA_BENCH_TINY="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--layers", "1", "--vocab", "4096"], capture_output=True, text=True,
                         env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
              "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in d, k
    assert d["impl"] == "reference" and d["cpu_baseline"]["kind"] in ("reference", "port")
    assert d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["extrapolated"] is False      # --steps 1: whole step
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["value"] > 0 and d["vs_baseline"] is None

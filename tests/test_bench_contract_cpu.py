"""CPU: the benchmark's CPU arm and JSON contract on a tiny workload (no GPU involved)."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_cpu_sample_scales_to_the_full_workload():
    import bench
    from ancora_cutile_b200 import shapes as S
    shp = S.qwen3_0_6b_shapes(n_layers=3, hidden=128, q_heads=2, kv_heads=1, head_dim=128, ffn=384, vocab=2048)
    mu = bench.route(shp)
    assert len(mu) == 21
    step, muon_scale, adamw_scale, nsel, n = bench.cpu_sample_step(shp, mu, layers=1, adamw_elems=1 << 14)
    assert nsel == 7 and abs(muon_scale - 3.0) < 1e-9                      # 1 of 3 identical layers
    a_total = sum(int(np.prod(s)) for k, s in shp.items() if k not in set(mu))
    assert abs(adamw_scale - a_total / (1 << 14)) < 1e-9
    tm, ta = step()
    assert tm > 0 and ta > 0


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
    assert d["impl"] == "reference" and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["value"] > 0 and d["vs_baseline"] is None

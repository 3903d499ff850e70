"""Generates the golden fixtures in this directory by running the REFERENCE's own
Python code (ancora-cutile checked out at the path given on the command line).

    python tests/golden/make_golden.py /path/to/ancora-cutile

The reference imports ``cuda.core`` at module scope (ancora/kernels/loss.py:30) but
uses nothing from it at import time, so an empty stand-in module is registered
before importing.  Only host (numpy) code of the reference is executed:

* ancora.optim.muon.newton_schulz5            -> ns_keller.npz
* tests/kernels/_probe_polar_express.ns + PE  -> ns_pe.npz
* ancora.optim.muon.Muon (3 steps)            -> host_muon.npz
* ancora.optim.adamw._bf16_bits/_bits_f32,
  ancora.optim.muon._bf                       -> bf16.npz
* ancora.kernels.muon_ns.PE_SCHEDULE/_coef_at,
  ancora.optim.hybrid.default_is_muon         -> tables.json
* ancora.kernels.quant._e4m3_table/f32_to_e4m3/
  dequantize_rowblock (host helpers)          -> e4m3.npz

* the four arithmetic statements of the
  ancora.optim.adamw._adamw kernel body,
  read from the source file and evaluated on
  float32 numpy arrays                        -> adamw.npz
  the same statements on zeros, signed zeros, denormals, infinities and NaNs
                                              -> adamw_special.npz

The reference's AdamW runs only on a GPU (cuda.tile kernel) and has no host function to
call.  Its arithmetic is four statements of plain operator syntax (adamw.py:34-37), so the
generator reads those statements from the checkout and executes their text with numpy
float32 arrays for the tiles, numpy float32 scalars for the runtime scalars and
``ct.sqrt = numpy.sqrt``: operator precedence and association are then the reference's own
text, not a reading of it.  A change of operation order in the reference changes adamw.npz.
"""
import importlib.util
import json
import os
import re
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.modules.setdefault("cuda.core", types.ModuleType("cuda.core"))
    from ancora.optim.muon import newton_schulz5, Muon, _bf
    from ancora.optim.adamw import _bf16_bits, _bits_f32
    from ancora.optim.hybrid import default_is_muon
    from ancora.kernels.muon_ns import PE_SCHEDULE, _coef_at, A_COEF, B_COEF, C_COEF

    spec = importlib.util.spec_from_file_location(
        "_probe_pe", os.path.join(ref_root, "tests", "kernels", "_probe_polar_express.py"))
    probe = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(probe)

    rng = np.random.default_rng(20240607)

    # 1. Keller fp32 Newton-Schulz, wide / tall / square
    out = {}
    for i, shp in enumerate([(128, 256), (256, 128), (128, 128)]):
        G = (rng.standard_normal(shp) * 1e-3).astype(np.float32)
        out[f"in{i}"] = G
        out[f"out{i}"] = newton_schulz5(G, 5)
    np.savez_compressed(os.path.join(HERE, "ns_keller.npz"), **out)

    # 2. Polar-Express fp32 Newton-Schulz (host probe's ns())
    out = {}
    for i, shp in enumerate([(128, 256), (128, 128)]):
        X = (rng.standard_normal(shp) @ np.diag(rng.uniform(0.1, 3.0, shp[1]))).astype(np.float32)
        out[f"in{i}"] = X
        out[f"out{i}"] = probe.ns(X, probe.PE, 5).astype(np.float32)
        out[f"out{i}_n7"] = probe.ns(X, probe.PE, 7).astype(np.float32)   # tail triple repeats
    np.savez_compressed(os.path.join(HERE, "ns_pe.npz"), **out)

    # 3. host Muon, 3 steps, one tall and one wide weight
    P = {"tall": (rng.standard_normal((256, 128)) * 0.02).astype(np.float32),
         "wide": (rng.standard_normal((128, 256)) * 0.02).astype(np.float32)}
    opt = Muon(P, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5)
    out = {f"p_{k}": v for k, v in P.items()}
    for t in range(3):
        g = {k: (rng.standard_normal(v.shape) * 1e-3).astype(np.float32) for k, v in P.items()}
        for k, v in g.items():
            out[f"g{t}_{k}"] = v
        opt.step(g)
    for k in P:
        out[f"master_{k}"] = opt.master()[k]
        out[f"weights_{k}"] = opt.weights()[k]
        out[f"buf_{k}"] = opt.buf[k]
    np.savez_compressed(os.path.join(HERE, "host_muon.npz"), **out)

    # 4. bf16 rounding helpers (ties, subnormals, infinities, signed zeros, random)
    edge = np.array([0.0, -0.0, 1.0, -1.0, 1.00390625, 1.01171875, 1.0078125, 3.0e38, -3.0e38,
                     3.3895314e38, np.inf, -np.inf, 1e-40, -1e-40, 1.17549435e-38, 65504.0],
                    dtype=np.float32)
    ties = (np.arange(0x3F800000, 0x3F800000 + 8 * 0x8000, 0x8000, dtype=np.uint32)).view(np.float32)
    x = np.concatenate([edge, ties, (rng.standard_normal(4096) * 0.02).astype(np.float32)])
    bits = _bf16_bits(x)
    np.savez_compressed(os.path.join(HERE, "bf16.npz"), x=x, bits=bits, back=_bits_f32(bits), bf=_bf(x))

    # 5. tables
    names = (["embed", "final_norm", "lm_head"] +
             [f"layers.{l}.{n}" for l in range(2) for n in
              ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj",
               "input_ln", "post_ln", "q_norm", "k_norm", "router", "experts.3.gate_proj")])
    two_d = lambda n: not any(t in n for t in ("_ln", "norm"))
    routing = {n: bool(default_is_muon(n, np.zeros((2, 2) if two_d(n) else (2,)))) for n in names}
    tables = {
        "keller": [A_COEF, B_COEF, C_COEF],
        "pe_schedule": [list(t) for t in PE_SCHEDULE],
        "coef_at_pe": [list(_coef_at(PE_SCHEDULE, k)) for k in range(8)],
        "coef_at_none": [list(_coef_at(None, k)) for k in range(3)],
        "routing": routing,
    }
    with open(os.path.join(HERE, "tables.json"), "w") as f:
        json.dump(tables, f, indent=1, sort_keys=True)

    # 6. E4M3 / MXFP8 host helpers of ancora/kernels/quant.py (its own generator, so the files
    #    above do not depend on this section): the 256-entry decode table, the host rounding
    #    f32_to_e4m3 (nearest, ties to the smaller magnitude: it differs from the device
    #    conversion's ties-to-even only at exact ties) and dequantize_rowblock
    from ancora.kernels.quant import _e4m3_table, f32_to_e4m3, dequantize_rowblock
    rq = np.random.default_rng(77)
    w = (rq.standard_normal(8192) * np.exp(rq.uniform(-4, 6, 8192))).astype(np.float32)
    w16 = _bits_f32(_bf16_bits(w))                               # bf16-valued inputs: many exact ties
    xq = np.concatenate([w, w16, np.array([0.0, -0.0, 448.0, -448.0, 464.0, 1e9, 2.0 ** -9, 2.0 ** -10,
                                           3 * 2.0 ** -10], np.float32)])
    fp8 = rq.integers(0, 256, (64, 64)).astype(np.uint8)
    fp8[(fp8 & 0x7F) == 0x7F] = 0x7E                             # no NaN codes
    sc = rq.integers(100, 140, (64, 2)).astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "e4m3.npz"), table=_e4m3_table(), x=xq, bytes=f32_to_e4m3(xq),
                        fp8=fp8, scale=sc, dequant=dequantize_rowblock(fp8, sc).astype(np.float32))
    # 7. AdamW: the kernel body's arithmetic statements, executed as written
    text = open(os.path.join(ref_root, "ancora", "optim", "adamw.py")).read().splitlines()
    body = [l.strip() for l in text if re.match(r"\s+(mn|vn|upd|pn)\s*=", l)]
    assert [l.split("=")[0].strip() for l in body] == ["mn", "vn", "upd", "pn"], body
    ra = np.random.default_rng(0)
    n = 1 << 14
    f = np.float32
    p = (ra.standard_normal(n) * 0.02).astype(f)
    m = (ra.standard_normal(n) * 1e-4).astype(f)
    v = np.abs(ra.standard_normal(n) * 1e-6).astype(f)
    g = _bits_f32(_bf16_bits((ra.standard_normal(n) * 1e-3).astype(f))).astype(f)      # bf16-valued gradient
    p[:8] = [0.0, -0.0, 1.0, -1.0, 3e38, -3e38, 1e-30, 65504.0]
    v[:4] = [0.0, 1e-38, 1e10, 1e-12]
    g[4:8] = [0.0, 1.0, -1.0, 1e-20]
    lr, b1, b2, eps, wd, t = 3e-4, 0.9, 0.95, 1e-8, 0.1, 10
    env = dict(ct=types.SimpleNamespace(sqrt=np.sqrt), g=g, tm=m, tv=v, tp=p,
               beta1=f(b1), beta2=f(b2), eps=f(eps), lr=f(lr), wd=f(wd),
               ibc1=f(1.0 / (1.0 - b1 ** t)), ibc2=f(1.0 / (1.0 - b2 ** t)))   # scalars as adamw.py:90-97 passes them
    with np.errstate(all="ignore"):
        for stmt in body:
            exec(stmt, env)
    for k in ("mn", "vn", "pn"):
        assert env[k].dtype == np.float32, (k, env[k].dtype)
    np.savez_compressed(os.path.join(HERE, "adamw.npz"), p=p, m=m, v=v, g=g,
                        hyper=np.array([lr, b1, b2, eps, wd, t], np.float64),
                        mn=env["mn"], vn=env["vn"], pn=env["pn"], p16=_bf16_bits(env["pn"]),
                        statements=np.array(body))
    # 8. The same statements on special operands (rows no token touched: g = m = v = 0; signed zeros;
    #    denormal, infinite and NaN moments and gradients)
    n = 64
    p = (ra.standard_normal(n) * 0.02).astype(f)
    m = (ra.standard_normal(n) * 1e-4).astype(f)
    v = np.abs(ra.standard_normal(n) * 1e-6).astype(f)
    g = _bits_f32(_bf16_bits((ra.standard_normal(n) * 1e-3).astype(f))).astype(f)
    g[0:8] = 0.0; m[0:8] = 0.0; v[0:8] = 0.0
    g[8:16] = -0.0; m[8:16] = 0.0; v[8:16] = 0.0
    m[16:24] = -0.0; g[16:24] = 0.0
    v[24:28] = np.inf; g[24:28] = 0.0; m[24:28] = 0.0
    v[28:32] = np.nan; g[28:32] = 0.0; m[28:32] = 0.0
    g[32:36] = np.nan
    m[36:40] = np.inf
    v[40:44] = f(1e-42)
    g[44:48] = f(1e-30); m[44:48] = 0.0; v[44:48] = 0.0
    env = dict(ct=types.SimpleNamespace(sqrt=np.sqrt), g=g, tm=m, tv=v, tp=p,
               beta1=f(b1), beta2=f(b2), eps=f(eps), lr=f(lr), wd=f(wd),
               ibc1=f(1.0 / (1.0 - b1 ** t)), ibc2=f(1.0 / (1.0 - b2 ** t)))
    with np.errstate(all="ignore"):
        for stmt in body:
            exec(stmt, env)
    np.savez_compressed(os.path.join(HERE, "adamw_special.npz"), p=p, m=m, v=v, g=g,
                        hyper=np.array([lr, b1, b2, eps, wd, t], np.float64),
                        mn=env["mn"], vn=env["vn"], pn=env["pn"])
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/ancora-cutile")
    main(sys.argv[1])

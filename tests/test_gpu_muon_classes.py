"""GPU: the Muon classes against the reference's host Muon restated in the oracle.

Tolerances from tests/kernels/_probe_device_muon.py:63-65,131-133 (after 5 steps the total
update has cos > 0.99 and rel < 0.06 vs the fp32 host optimizer, for square / wide / tall) and
tests/training/test_batched_proj_muon.py:71-74 (batched == per-weight, scope == global bitwise)."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import muon_ref

pytestmark = pytest.mark.gpu
SHAPES = {"sq": (256, 256), "wide": (128, 384), "tall": (384, 128)}


def cos_rel(a, b):
    a, b = a.ravel().astype(np.float64), b.ravel().astype(np.float64)
    return (float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30)),
            float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30)))


def _setup(rng):
    P = {n: (rng.standard_normal(s) * 0.02).astype(np.float32) for n, s in SHAPES.items()}
    Gs = [{n: (rng.standard_normal(s) * 1e-3).astype(np.float32) for n, s in SHAPES.items()} for _ in range(5)]
    return P, Gs


def test_host_api_muon_vs_host_reference(ctx):
    rng = np.random.default_rng(0)
    P, Gs = _setup(rng)
    opt = anc.Muon(P, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, ctx=ctx)     # Keller default
    ref = muon_ref.HostMuon(P, schedule=None)
    for g in Gs:
        opt.step(g, None)
        ref.step(g)
    m = opt.master()
    for n in P:
        c, r = cos_rel(m[n] - P[n], ref.w[n] - P[n])
        assert c > 0.99 and r < 0.06, (n, c, r)
        assert np.array_equal(f32_to_bf16_bits(opt.weights()[n]), f32_to_bf16_bits(m[n]))   # weights == RNE(master)
    opt.free()


def _resident_weights(ctx, P, G):
    ws = []
    for lid, n in enumerate(P):
        K, N = P[n].shape
        ws.append(dict(buf=anc.DBuf.zeros((K, N), np.float32, ctx), p32=anc.DBuf(P[n], ctx),
                       p16=anc.DBuf(f32_to_bf16_bits(P[n]), ctx), G=anc.DBuf(G[n], ctx), K=K, N=N, lid=lid, name=n))
    return ws


def _free(ws):
    for w in ws:
        for k in ("buf", "p32", "p16", "G"):
            w[k].free()


def test_batched_equals_per_weight_and_scope_bitwise(ctx):
    rng = np.random.default_rng(1)
    P = {f"l{i}.{n}": (rng.standard_normal(s) * 0.02).astype(np.float32)
         for i in range(3) for n, s in SHAPES.items()}
    G = {n: (rng.standard_normal(p.shape) * 1e-3).astype(np.float32) for n, p in P.items()}
    results = []
    for mode in ("global", "scope1", "chunk2", "per_weight"):
        ws = _resident_weights(ctx, P, G)
        for i, w in enumerate(ws):
            w["lid"] = i // 3
        if mode == "per_weight":
            opts = [anc.ResidentMuon(w["p32"], w["p16"], w["K"], w["N"], None, ctx=ctx) for w in ws]
            for _ in range(3):
                for o, w in zip(opts, ws):
                    o.step(w["G"], ctx.stream, 0.02)
        else:
            kw = dict(scope=1) if mode == "scope1" else dict(chunk=2) if mode == "chunk2" else {}
            bp = anc.BatchedProjMuon(ws, **kw, ctx=ctx)
            for _ in range(3):
                bp.step(ctx.stream, 0.02)
            opts = [bp]
        ctx.sync()
        assert ctx.status() == 0
        results.append({w["name"]: (w["p32"].to_numpy(), w["p16"].to_numpy()) for w in ws})
        for o in opts:
            o.free()
        _free(ws)
    base = results[0]
    for other in results[1:]:
        for n in base:
            assert np.array_equal(base[n][0], other[n][0]), n
            assert np.array_equal(base[n][1], other[n][1]), n


def test_resident_muon_vs_host_reference_pe(ctx):
    rng = np.random.default_rng(2)
    P, Gs = _setup(rng)
    prev = anc.set_polar_express(True)
    try:
        ref = muon_ref.HostMuon(P, schedule=muon_ref.PE_SCHEDULE)
        ws = _resident_weights(ctx, P, Gs[0])
        bp = anc.BatchedProjMuon(ws, ctx=ctx)
        for g in Gs:
            for w in ws:
                w["G"].upload(g[w["name"]])
            bp.step(ctx.stream, 0.02)
            ref.step(g)
        ctx.sync()
        for w in ws:
            n = w["name"]
            c, r = cos_rel(w["p32"].to_numpy() - P[n], ref.w[n] - P[n])
            assert c > 0.99 and r < 0.06, (n, c, r)
            assert np.array_equal(w["p16"].to_numpy(), f32_to_bf16_bits(w["p32"].to_numpy()))
        bp.free()
        _free(ws)
    finally:
        anc.set_polar_express(bool(prev))


def test_misaligned_shape_raises(ctx):
    with pytest.raises(AssertionError):
        anc.Muon({"router": np.zeros((1024, 16), np.float32)}, ctx=ctx)
    with pytest.raises(AssertionError):
        anc.Muon({"gain": np.zeros((128,), np.float32)}, ctx=ctx)


@pytest.mark.parametrize("shape", [(512, 512), (1024, 512)])
def test_descends_on_a_quadratic_like_the_host_optimizer(ctx, shape):
    """Minimise 0.5 * ||W - T||^2 with g = W - T for 30 steps from W = 0: the loss must fall below
    0.2 of its start and stay within 3x the host optimizer's ratio + 0.05
    (tests/kernels/_probe_device_muon.py:72-100, square and tall)."""
    K, N = shape
    rng = np.random.default_rng(1)
    T = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    host = muon_ref.HostMuon({"w": np.zeros(shape, np.float32)}, schedule=None)
    dev = anc.Muon({"w": np.zeros(shape, np.float32)}, lr=0.02, momentum=0.95, ns_steps=5, schedule=None, ctx=ctx)
    lh, ld = [], []
    for _ in range(30):
        g = host.w["w"] - T
        lh.append(0.5 * float(np.sum(g * g)))
        host.step({"w": g})
        g = dev.master()["w"] - T
        ld.append(0.5 * float(np.sum(g * g)))
        dev.step({"w": g}, None)
    dev.free()
    drop_d, drop_h = ld[-1] / ld[0], lh[-1] / lh[0]
    assert drop_d < 0.2 and drop_d < 3 * drop_h + 0.05, (drop_d, drop_h)


def test_interleaved_weights_of_three_shapes_do_not_contaminate_each_other(ctx):
    """Square, wide and tall ResidentMuon objects built over one MuonScratch and stepped in turn
    within every step, each against its own host optimizer (tests/kernels/_probe_device_muon.py:104-138:
    shared scratch, transposed path, cos > 0.99, rel < 0.06 after 5 steps)."""
    shapes = [(256, 256), (256, 512), (512, 256)]
    rng = np.random.default_rng(0)
    sc = anc.MuonScratch(shapes)
    items = []
    for K, N in shapes:
        W0 = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
        p32, p16 = anc.DBuf(W0, ctx), anc.DBuf(f32_to_bf16_bits(W0), ctx)
        g_dev = anc.DBuf.zeros((K, N), np.float32, ctx)
        items.append((W0, muon_ref.HostMuon({"w": W0.copy()}, schedule=None), p32, p16,
                      anc.ResidentMuon(p32, p16, K, N, sc, schedule=None, ctx=ctx), g_dev))
    for _ in range(5):
        for W0, host, p32, p16, rm, g_dev in items:
            g = rng.standard_normal(W0.shape).astype(np.float32)
            host.step({"w": g})
            g_dev.upload(g)
            rm.step(g_dev, ctx.stream, 0.02)
    ctx.sync()
    assert ctx.status() == 0
    for W0, host, p32, p16, rm, g_dev in items:
        c, r = cos_rel(W0 - p32.to_numpy(), W0 - host.w["w"])
        assert c > 0.99 and r < 0.06, (W0.shape, c, r)
        assert np.array_equal(p16.to_numpy(), f32_to_bf16_bits(p32.to_numpy()))
        rm.free()
        for b in (p32, p16, g_dev):
            b.free()
    sc.free()

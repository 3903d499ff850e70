"""GPU: the benchmark configurations at their full sizes.

AdamW case: AdamW on one 151936x1024 tensor, bf16 grads, step 10, SR seed 1234 -- the device
result must equal the oracle bit for bit on all 155,582,464 elements (fp32 state and bf16 copy).
MoE expert shape: a batch of 16 rectangular experts (768x1024) through the whole Muon step, each
compared with its own fp32 host result, plus the size-independent property that the bf16
Newton-Schulz output is close to orthogonal."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import adamw_ref, bf16 as obf, muon_ref

pytestmark = pytest.mark.gpu


def test_config1_full_size_bit_exact(ctx):
    V, H = 151936, 1024
    n = V * H
    rng = np.random.default_rng(0)
    p = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    m = rng.standard_normal(n, dtype=np.float32) * np.float32(1e-4)
    v = np.abs(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-6))
    g16 = f32_to_bf16_bits(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3))
    t = dict(g=anc.DBuf(g16, ctx), p32=anc.DBuf(p, ctx), m=anc.DBuf(m, ctx), v=anc.DBuf(v, ctx),
             p16=anc.DBuf.zeros((n,), np.uint16, ctx), numel=n, wd=0.1)
    opt = anc.ResidentAdamW([t], grad_dtype="bf16", rounding="sr", seed=1234, ctx=ctx)
    opt.step(None, lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, t=10)
    ctx.sync()
    assert ctx.status() == 0
    s = adamw_ref.adamw_scalars(3e-4, 0.9, 0.95, 1e-8, 10)
    pn, mn, vn, p16 = adamw_ref.adamw_step(p, m, v, bits_to_f32(g16), s, 0.1, "sr", 1234, 10, 0)
    assert np.array_equal(t["m"].to_numpy(), mn)
    assert np.array_equal(t["v"].to_numpy(), vn)
    assert np.array_equal(t["p32"].to_numpy(), pn)
    assert np.array_equal(t["p16"].to_numpy(), p16)
    # the stochastic copy differs from round-to-nearest in a large share of the elements
    # and never by more than one bf16 step
    rne = obf.rne_bits(pn)
    d = p16.astype(np.int32) - rne.astype(np.int32)
    assert 0.2 < np.mean(d != 0) < 0.8 and np.abs(d).max() <= 1
    opt.free()
    for k in ("g", "p32", "m", "v", "p16"):
        t[k].free()


def test_moe_expert_batch_full_muon_step(ctx):
    E, K, N = 16, 1024, 768          # gate/up experts (H, Ie): tall -> NS runs on (768,1024)
    rng = np.random.default_rng(5)
    ws, P, G = [], [], []
    for e in range(E):
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        g = obf.rne_f32((rng.standard_normal((K, N)) * 1e-3).astype(np.float32))
        P.append(w); G.append(g)
        ws.append(dict(buf=anc.DBuf.zeros((K, N), np.float32, ctx), p32=anc.DBuf(w, ctx),
                       p16=anc.DBuf(f32_to_bf16_bits(w), ctx), G=anc.DBuf(f32_to_bf16_bits(g), ctx), K=K, N=N))
    bp = anc.BatchedProjMuon(ws, grad_dtype="bf16", schedule=anc.PE_SCHEDULE, ctx=ctx)
    bp.step(ctx.stream, 0.02)
    ctx.sync()
    assert ctx.status() == 0
    lr_scale = np.float32(0.02 * muon_ref.shape_scale(K, N))
    for e in (0, 7, 15):
        _, u = muon_ref.momentum(np.zeros((K, N), np.float32), G[e], 0.95)
        o = muon_ref.ns_fp32(obf.rne_f32(u), 5, muon_ref.PE_SCHEDULE)
        got = (P[e] - ws[e]["p32"].to_numpy()) / lr_scale           # the device's orthogonalised update
        rel = np.linalg.norm(got - o) / np.linalg.norm(o)
        assert rel < 2e-2, (e, rel)
        ot = got.T                                                   # (768, 1024): rows ~ orthonormal
        err = np.linalg.norm(ot @ ot.T - np.eye(N, dtype=np.float32)) / np.sqrt(N)
        assert err < 0.35, (e, err)                                  # PE-5 leaves sigma in ~[0.7, 1.2]
        assert np.array_equal(ws[e]["p16"].to_numpy(), f32_to_bf16_bits(ws[e]["p32"].to_numpy()))
    bp.free()
    for w in ws:
        for k in ("buf", "p32", "p16", "G"):
            w[k].free()

"""GPU: the reference's own parameter dicts and class names drop in.

* a dict shaped like MoEModel.params() (ancora/model/moe_model.py:51-60: 2-D attention and
  router tensors, 3-D expert stacks, embed, gains) goes through HybridOptimizer unmodified;
* DeviceMuon (ancora/optim/muon.py:88-135) and ExpertMuonScratch
  (ancora/kernels/moe.py:404-421) exist with the reference's signatures;
* ``opt.muon`` / ``opt.adamw`` step on their own (ancora/optim/hybrid.py:40-47);
* the MoE family (BASELINE config 5 shapes, fewer layers): batched expert Newton-Schulz
  against the fp32 chain, bitwise equal across batch sizes and ZeRO-1 world sizes.
"""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import muon_ns, shapes as S
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from ancora_cutile_b200.hybrid import muon_names_for
from oracle import adamw_ref, bf16 as obf, muon_ref

pytestmark = pytest.mark.gpu
AKW = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1)


def moe_model_params(rng, layers=2, H=256, E=4, Ie=128, vocab=512):
    """Names and ranks of MoEModel.params(): 'layerI.<attn>', 'layerI.ffn.<ffn>'."""
    W = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)
    p = {"embed": W(vocab, H), "final_norm": np.ones(H, np.float32)}
    for i in range(layers):
        p[f"layer{i}.input_ln"] = np.ones(H, np.float32)
        p[f"layer{i}.q_proj"] = W(H, 2 * 128)
        p[f"layer{i}.k_proj"] = W(H, 128)
        p[f"layer{i}.v_proj"] = W(H, 128)
        p[f"layer{i}.o_proj"] = W(2 * 128, H)
        p[f"layer{i}.post_ln"] = np.ones(H, np.float32)
        p[f"layer{i}.ffn.router"] = W(H, E)                 # 2-D, but (256, 4) cannot be tiled
        p[f"layer{i}.ffn.gate_proj"] = W(E, H, Ie)
        p[f"layer{i}.ffn.up_proj"] = W(E, H, Ie)
        p[f"layer{i}.ffn.down_proj"] = W(E, Ie, H)
    return p


@pytest.mark.parametrize("expert_muon", [False, True])
def test_moe_model_param_dict_goes_through_unmodified(ctx, expert_muon):
    rng = np.random.default_rng(0)
    params = moe_model_params(rng)
    prev = anc.set_polar_express(True)
    try:
        opt = anc.HybridOptimizer(params, adamw_kw=AKW, grad_dtype="f32", expert_muon=expert_muon, ctx=ctx)
        r = opt.routing()
        assert set(r) == {"muon", "adamw"}
        assert opt.muon_fallback == ["layer0.ffn.router", "layer1.ffn.router"]
        assert all(n in r["adamw"] for n in opt.muon_fallback)              # the router is under AdamW
        assert ("layer0.ffn.gate_proj" in r["muon"]) == expert_muon          # 3-D stacks: AdamW unless asked
        assert "layer1.q_proj" in r["muon"] and "embed" in r["adamw"]
        grads = {n: (rng.standard_normal(p.shape) * 1e-3).astype(np.float32) for n, p in params.items()}
        opt.step(grads, None)
        w, master = opt.weights(), opt.master()
        assert set(w) == set(params) and all(w[n].shape == params[n].shape for n in params)
        # AdamW-routed tensors (router included): bit-exact against the oracle
        s = adamw_ref.adamw_scalars(AKW["lr"], *AKW["betas"], AKW["eps"], 1)
        for n in r["adamw"]:
            p = params[n].reshape(-1)
            z = np.zeros_like(p)
            pn, _, _, p16 = adamw_ref.adamw_step(p, z, z, grads[n].reshape(-1), s,
                                                 0.0 if params[n].ndim == 1 else AKW["wd"], "rne")
            assert np.array_equal(master[n].reshape(-1), pn), n
            assert np.array_equal(f32_to_bf16_bits(w[n]).reshape(-1), p16), n
        # Muon-routed tensors: update within the reference's bar of the fp32 host step
        for n in r["muon"]:
            mats = [(params[n], grads[n], master[n])] if params[n].ndim == 2 else \
                [(params[n][e], grads[n][e], master[n][e]) for e in range(params[n].shape[0])]
            for W0, g, got in mats:
                _, u = muon_ref.momentum(np.zeros_like(W0), g, 0.95)
                o = muon_ref.ns_fp32(obf.rne_f32(u), 5, muon_ref.PE_SCHEDULE)
                want = -np.float32(0.02 * muon_ref.shape_scale(*W0.shape)) * o
                rel = np.linalg.norm((got - W0) - want) / np.linalg.norm(want)
                assert rel < 2e-2, (n, rel)
        opt.free()
    finally:
        anc.set_polar_express(bool(prev))


def test_parts_step_on_their_own_like_the_combined_step(ctx):
    shp = S.qwen3_0_6b_shapes(n_layers=1, hidden=128, q_heads=2, kv_heads=1, head_dim=128, ffn=256, vocab=512)
    params = S.synthetic_params(shp, seed=2)
    rng = np.random.default_rng(3)
    grads = [{n: (rng.standard_normal(s) * 1e-3).astype(np.float32) for n, s in shp.items()} for _ in range(2)]
    a = anc.HybridOptimizer(params, adamw_kw=AKW, ctx=ctx)
    b = anc.HybridOptimizer(params, adamw_kw=AKW, ctx=ctx)
    for g in grads:
        a.step(g, None)
        b.muon.step({n: g[n] for n in b.muon_names}, None)
        b.adamw.step({n: g[n] for n in b.adamw_names}, None)
    assert a.adamw.t == b.adamw.t == 2 and a.muon.t == b.muon.t == 2
    wa, wb, ma, mb = a.weights(), b.weights(), a.master(), b.master()
    for n in shp:
        assert np.array_equal(wa[n], wb[n]) and np.array_equal(ma[n], mb[n]), n
    assert set(b.muon.weights()) == set(b.muon_names) and set(b.adamw.master()) == set(b.adamw_names)
    b.muon.lr = 0.01
    assert b.engine.muon_kw["lr"] == 0.01
    b.muon.free(); b.adamw.free()                       # no-ops: the arenas belong to the hybrid
    a.free(); b.free()


def test_device_muon_and_expert_scratch(ctx):
    rng = np.random.default_rng(4)
    prev = anc.set_polar_express(True)
    try:
        for shape in ((256, 128), (128, 384)):
            W = (rng.standard_normal(shape) * 0.02).astype(np.float32)
            g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
            dm = anc.DeviceMuon(W, lr=0.02, momentum=0.95, ns_steps=5, ctx=ctx)
            assert (dm.K, dm.N, dm.tr) == (shape[0], shape[1], shape[0] > shape[1])
            assert abs(dm.lr_scale - 0.02 * max(1.0, shape[0] / shape[1]) ** 0.5) < 1e-12
            gd = anc.DBuf(g, ctx)
            dm.step(gd, ctx.stream)
            ctx.sync()
            ref = muon_ref.HostMuon({"w": W}, schedule=muon_ref.PE_SCHEDULE)
            ref.step({"w": g})
            a, b = (dm.master() - W).ravel(), (ref.w["w"] - W).ravel()
            assert np.linalg.norm(a - b) / np.linalg.norm(b) < 2e-2
            assert np.array_equal(f32_to_bf16_bits(dm.weights()), f32_to_bf16_bits(dm.master()))
            dm.free(); gd.free()
        # the expert scratch, driven the way GroupedMoEFFN.step drives it (kernels/moe.py:583-586)
        E, M = 3, 256
        sc = anc.ExpertMuonScratch(E, M, ctx=ctx)
        assert sc.u.shape == (E * M, M) and sc.recip.shape == (E, 1) and sc.nbytes() > 0
        U = f32_to_bf16_bits((rng.standard_normal((E * M, M)) * 1e-3).astype(np.float32))
        outs = []
        for fused in (True, False):                     # fused=False: one launch per phase, same bits
            sc.u.upload(U)
            muon_ns.newton_schulz_resident_e(sc.u, sc.gA, sc.gA2, sc.gB, sc.gBX, sc.recip, E, M, M, ctx.stream,
                                             steps=5, schedule=muon_ns.PE_SCHEDULE, fused=fused)
            ctx.sync()
            outs.append(sc.u.to_numpy())
        assert np.array_equal(outs[0], outs[1])
        for e in range(E):
            want = muon_ref.ns_fp32(bits_to_f32(U[e * M:(e + 1) * M]), 5, muon_ref.PE_SCHEDULE)
            got = bits_to_f32(outs[0][e * M:(e + 1) * M])
            assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-2, e
        sc.free()
        assert ctx.status() == 0
    finally:
        anc.set_polar_express(bool(prev))


def test_moe_family_batched_experts(ctx):
    """4 layers of the MoE family (2 MoE layers x 16 experts x 3 tensors = 96 matrices of
    768x1024 in one Newton-Schulz batch): sampled experts against the fp32 chain, the whole step
    bitwise equal with batches of 8 and with the shards of a world of 4 built on this GPU."""
    shp = S.moe_family_shapes(n_layers=4, vocab=2048)
    mu = muon_names_for(shp)
    experts = [n for n in mu if ".experts." in n]
    assert len(experts) == 96 and all(sorted(shp[n]) == [768, 1024] for n in experts)
    assert all("router" not in n for n in mu)            # (1024, 16): AdamW
    params = S.synthetic_params(shp, seed=21)
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    grads = S.synthetic_grads_bf16(shp, seed=22)

    def run(rank=0, world=1, max_batch=0):
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=11,
                                 rank=rank, world=world, schedule=anc.PE_SCHEDULE, max_batch=max_batch, ctx=ctx)
        eng.upload_grads(grads, ctx.stream)
        eng.step(ctx.stream, exchange=False)
        ctx.sync()
        assert ctx.status() == 0
        bits, _ = eng.download_weights_bits()
        out = ({n: b.copy() for n, b in bits.items()}, eng.master(), {n: eng.owned_range(n) for n in shp})
        eng.free()
        return out

    full_bits, full_master, _ = run()
    for n in experts[::8]:                               # every 8th expert matrix vs the fp32 chain
        g = bits_to_f32(grads[n])
        _, u = muon_ref.momentum(np.zeros(shp[n], np.float32), g, 0.95)
        o = muon_ref.ns_fp32(obf.rne_f32(u), 5, muon_ref.PE_SCHEDULE)
        want = -np.float32(0.02 * muon_ref.shape_scale(*shp[n])) * o
        got = full_master[n][2].reshape(shp[n]) - params[n]
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel < 2e-2, (n, rel)
    bits8, master8, _ = run(max_batch=8)
    for n in shp:
        assert np.array_equal(bits8[n], full_bits[n]) and np.array_equal(master8[n][2], full_master[n][2]), n
    for r in range(4):
        bits, master, owned = run(r, 4)
        for n in shp:
            s, e = owned[n]
            if e > s:
                assert np.array_equal(bits[n].reshape(-1)[s:e], full_bits[n].reshape(-1)[s:e]), (r, n)
                assert np.array_equal(master[n][2], full_master[n][2][s:e]), (r, n)

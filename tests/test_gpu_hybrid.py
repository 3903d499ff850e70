"""GPU: the hybrid optimizer end to end on a small model, and ZeRO-1 sharding.

ZeRO-1 is checked on ONE GPU by building the rank-r engine of a world of 2 and of 4 one
after another (no collective): the bf16 parameters each rank owns and its fp32 state must
equal the single-GPU engine's bit for bit."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import shapes as S
from ancora_cutile_b200.bf16 import f32_to_bf16_bits
from oracle import adamw_ref, bf16 as obf, muon_ref

pytestmark = pytest.mark.gpu
AKW = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1)


def small_shapes():
    return S.qwen3_0_6b_shapes(n_layers=2, hidden=128, q_heads=2, kv_heads=1, head_dim=128, ffn=384, vocab=1000)


def test_routing_matches_reference_rule():
    shp = S.qwen3_0_6b_shapes()
    params = {n: np.empty((0,) * len(s)) for n, s in shp.items()}
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    assert len(mu) == 196 and len(shp) - len(mu) == 114
    assert sum(int(np.prod(shp[n])) for n in shp if n not in mu) == 155_648_000


def test_hybrid_step_vs_oracle(ctx):
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=0)
    rng = np.random.default_rng(1)
    prev = anc.set_polar_express(True)
    try:
        opt = anc.HybridOptimizer(params, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=1234, ctx=ctx)
        r = opt.routing()
        assert len(r["muon"]) == 14 and "embed" in r["adamw"]
        ref_mu = muon_ref.HostMuon({n: params[n] for n in r["muon"]}, schedule=muon_ref.PE_SCHEDULE)
        st = {n: [params[n].reshape(-1).copy(), np.zeros(params[n].size, np.float32), np.zeros(params[n].size, np.float32)]
              for n in r["adamw"]}
        for t in range(1, 4):
            grads = {n: obf.rne_f32((rng.standard_normal(s) * 1e-3).astype(np.float32)) for n, s in shp.items()}
            opt.step(grads, None)
            ref_mu.step({n: grads[n] for n in r["muon"]})
            s = adamw_ref.adamw_scalars(AKW["lr"], *AKW["betas"], AKW["eps"], t)
            p16 = {}
            for n in r["adamw"]:
                wd = 0.0 if len(shp[n]) == 1 else AKW["wd"]
                p, m, v, b = adamw_ref.adamw_step(*st[n], grads[n].reshape(-1), s, wd, "sr", 1234, t,
                                                  opt.engine.a_off[n])
                st[n] = [p, m, v]
                p16[n] = b
        master, w = opt.master(), opt.weights()
        for n in r["adamw"]:                                   # AdamW: bit-exact after 3 steps
            assert np.array_equal(master[n].reshape(-1), st[n][0]), n
            assert np.array_equal(f32_to_bf16_bits(w[n]).reshape(-1), p16[n]), n
        for n in r["muon"]:                                    # Muon: update within tolerance
            a, b = (master[n] - params[n]).ravel(), (ref_mu.w[n] - params[n]).ravel()
            rel = np.linalg.norm(a - b) / np.linalg.norm(b)
            assert rel < 0.06, (n, rel)
        opt.free()
    finally:
        anc.set_polar_express(bool(prev))


@pytest.mark.parametrize("world", [2, 4])
def test_zero1_shards_bitwise_equal_single(ctx, world):
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=3)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    grads = S.synthetic_grads_bf16(shp, seed=4)

    def run(rank, w):
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=7,
                                 rank=rank, world=w, schedule=anc.PE_SCHEDULE, ctx=ctx)
        for _ in range(2):
            eng.upload_grads(grads, ctx.stream)
            eng.step(ctx.stream, exchange=False)
        ctx.sync()
        assert ctx.status() == 0
        bits, _ = eng.download_weights_bits()
        bits = {n: b.copy() for n, b in bits.items()}
        res = (bits, eng.master(), {n: eng.owned_range(n) for n in shp})
        eng.free()
        return res

    full_bits, full_master, _ = run(0, 1)
    covered = {n: 0 for n in shp}
    for r in range(world):
        bits, master, owned = run(r, world)
        for n in shp:
            s, e = owned[n]
            if e <= s:
                continue
            covered[n] += e - s
            assert np.array_equal(bits[n].reshape(-1)[s:e], full_bits[n].reshape(-1)[s:e]), (r, n)
            ms, me, flat = master[n]
            assert (ms, me) == (s, e)
            assert np.array_equal(flat, full_master[n][2][s:e]), (r, n)
    for n, s in shp.items():
        assert covered[n] == int(np.prod(s)), n               # every element owned exactly once


def test_group_parts_leave_the_bits_unchanged(ctx, monkeypatch):
    """The largest shape group cut into two arena groups (what eight ranks do; forced here): the
    whole model on one GPU, the four shards of a world of 4 and the pipelined host round trip all
    give the bits of the uncut single-GPU step."""
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=3)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    grads = S.synthetic_grads_bf16(shp, seed=4)

    def run(rank, w, host=False):
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=7,
                                 rank=rank, world=w, schedule=anc.PE_SCHEDULE, ctx=ctx)
        n_groups = len(eng.groups)
        for _ in range(2):
            if host:
                eng.host_chunk_elems = 128 * 128 * 2
                eng.step_host(grads, ctx.stream)
            else:
                eng.upload_grads(grads, ctx.stream)
                eng.step(ctx.stream, exchange=False)
        ctx.sync()
        assert ctx.status() == 0
        bits, _ = eng.download_weights_bits()
        res = ({n: b.copy() for n, b in bits.items()}, eng.master(), {n: eng.owned_range(n) for n in shp}, n_groups)
        eng.free()
        return res

    full_bits, full_master, _, g_plain = run(0, 1)
    monkeypatch.setenv("ANCORA_GROUP_PARTS", "2")
    for host in (False, True):
        bits, master, _, g_cut = run(0, 1, host)
        assert g_cut == g_plain + 1
        for n in shp:
            assert np.array_equal(bits[n], full_bits[n]), (host, n)
            assert np.array_equal(master[n][2], full_master[n][2]), (host, n)
    for r in range(4):
        bits, master, owned, _ = run(r, 4)
        for n in shp:
            s, e = owned[n]
            if e > s:
                assert np.array_equal(bits[n].reshape(-1)[s:e], full_bits[n].reshape(-1)[s:e]), (r, n)
                assert np.array_equal(master[n][2], full_master[n][2][s:e]), (r, n)


def test_step_host_pipeline_equals_plain_step(ctx):
    """The pipelined host round trip (sub-chunked units on three streams) gives the same bits
    as upload + step + download, and its returned views are the updated parameters."""
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=5)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    g1, g2 = S.synthetic_grads_bf16(shp, seed=6), S.synthetic_grads_bf16(shp, seed=7)
    outs = []
    for mode in ("plain", "host", "host_tiny_chunks"):
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=9,
                                 schedule=anc.PE_SCHEDULE, ctx=ctx)
        if mode == "host_tiny_chunks":
            eng.host_chunk_elems = 128 * 128 * 2          # two small matrices per unit
        for g in (g1, g2):
            if mode == "plain":
                eng.upload_grads(g, ctx.stream)
                eng.step(ctx.stream)
                bits, _ = eng.download_weights_bits()
            else:
                bits, h2d, d2h = eng.step_host(g, ctx.stream)
                assert h2d == d2h and h2d > 0
        assert ctx.status() == 0
        outs.append(({n: b.copy() for n, b in bits.items()}, eng.master()))
        eng.free()
    for other in outs[1:]:
        for n in shp:
            assert np.array_equal(outs[0][0][n], other[0][n]), n
            assert np.array_equal(outs[0][1][n][2], other[1][n][2]), n


def test_state_dict_resume_is_bit_exact(ctx):
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=8)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    gs = [S.synthetic_grads_bf16(shp, seed=30 + k) for k in range(4)]
    mk = lambda p: anc.ResidentHybrid(p, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=21,
                                      schedule=anc.PE_SCHEDULE, ctx=ctx)
    a = mk(params)
    for g in gs[:2]:
        a.upload_grads(g, ctx.stream); a.step(ctx.stream)
    sd = a.state_dict()
    for g in gs[2:]:
        a.upload_grads(g, ctx.stream); a.step(ctx.stream)
    want_bits, _ = a.download_weights_bits()
    want_bits = {n: b.copy() for n, b in want_bits.items()}
    want_master = a.master()
    a.free()
    # a fresh engine built from unrelated initial values, then restored
    b = mk({n: np.zeros_like(p) for n, p in params.items()})
    b.load_state_dict(sd)
    assert b.t == 2
    for g in gs[2:]:
        b.upload_grads(g, ctx.stream); b.step(ctx.stream)
    got_bits, _ = b.download_weights_bits()
    for n in shp:
        assert np.array_equal(got_bits[n], want_bits[n]), n
        assert np.array_equal(b.master()[n][2], want_master[n][2]), n
    with pytest.raises(ValueError):
        sd2 = dict(sd); sd2["world"] = 2
        b.load_state_dict(sd2)
    b.free()


def test_graph_replay_equals_eager_steps(ctx):
    """One captured step replayed three times = three eager steps, bit for bit (the AdamW step
    number, bias corrections and SR stream advance inside the graph)."""
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=12)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    g = S.synthetic_grads_bf16(shp, seed=13)
    res = []
    for mode in ("eager", "graph"):
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=5,
                                 schedule=anc.PE_SCHEDULE, ctx=ctx)
        eng.upload_grads(g, ctx.stream)
        eng.step(ctx.stream)
        if mode == "graph":
            eng.capture_step(ctx.stream, horizon=8)
        for _ in range(3):
            eng.replay_step(ctx.stream) if mode == "graph" else eng.step(ctx.stream)
        ctx.sync()
        assert ctx.status() == 0 and eng.t == 4
        bits, _ = eng.download_weights_bits()
        res.append(({n: b.copy() for n, b in bits.items()}, eng.master()))
        eng.free()
    for n in shp:
        assert np.array_equal(res[0][0][n], res[1][0][n]), n
        assert np.array_equal(res[0][1][n][2], res[1][1][n][2]), n


def test_graph_replay_after_an_eager_step_and_a_restored_state(ctx):
    """The device step counter follows the host's: capture, eager step, replay must equal four
    eager steps; a state restored to an earlier step replays from there; a changed seed or a step
    outside the uploaded schedule asks for a new capture instead of using stale scalars."""
    shp = small_shapes()
    params = S.synthetic_params(shp, seed=14)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    g = S.synthetic_grads_bf16(shp, seed=15)

    def make():
        eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=5,
                                 schedule=anc.PE_SCHEDULE, ctx=ctx)
        eng.upload_grads(g, ctx.stream)
        return eng

    def snap(eng):
        ctx.sync()
        assert ctx.status() == 0
        bits, _ = eng.download_weights_bits()
        return {n: b.copy() for n, b in bits.items()}, eng.master()

    ref = make()
    for _ in range(2):
        ref.step(ctx.stream)
    sd2 = ref.state_dict()
    for _ in range(2):
        ref.step(ctx.stream)
    want = snap(ref)
    ref.free()

    eng = make()
    eng.step(ctx.stream)
    eng.capture_step(ctx.stream, horizon=8)
    eng.replay_step(ctx.stream)            # step 2
    eng.step(ctx.stream)                   # step 3, eager: the device counter is now behind
    eng.replay_step(ctx.stream)            # step 4
    assert eng.t == 4
    got = snap(eng)
    for n in shp:
        assert np.array_equal(got[0][n], want[0][n]) and np.array_equal(got[1][n][2], want[1][n][2]), n
    eng.load_state_dict(sd2)               # back to the state after step 2
    eng.replay_step(ctx.stream)
    eng.replay_step(ctx.stream)
    assert eng.t == 4
    got = snap(eng)
    for n in shp:
        assert np.array_equal(got[0][n], want[0][n]) and np.array_equal(got[1][n][2], want[1][n][2]), n
    eng.seed = 6
    with pytest.raises(RuntimeError):
        eng.replay_step(ctx.stream)
    eng.seed = 5
    eng.t = 100
    with pytest.raises(RuntimeError):
        eng.replay_step(ctx.stream)
    eng.free()

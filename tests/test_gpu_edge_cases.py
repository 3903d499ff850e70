"""GPU: edge cases of the host API and the bounded device waits."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import _lib as L
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import adamw_ref, bf16 as obf, muon_ref

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def test_default_hybrid_keeps_reference_semantics(ctx):
    """Defaults = the reference's: float32 grads, RNE copy, Keller coefficients, wd 0.01,
    no decay on 1-D tensors (ancora/optim/hybrid.py:29-43)."""
    rng = np.random.default_rng(0)
    params = {"embed": (rng.standard_normal((256, 128)) * 0.02).astype(np.float32),
              "layers.0.q_proj": (rng.standard_normal((128, 256)) * 0.02).astype(np.float32),
              "layers.0.input_ln": np.ones(128, np.float32), "lm_head": (rng.standard_normal((128, 256)) * 0.02).astype(np.float32)}
    opt = anc.HybridOptimizer(params, ctx=ctx)
    assert opt.routing() == {"muon": ["layers.0.q_proj"], "adamw": ["embed", "layers.0.input_ln", "lm_head"]}
    st = {n: [params[n].reshape(-1).copy(), np.zeros(params[n].size, np.float32), np.zeros(params[n].size, np.float32)]
          for n in opt.adamw_names}
    ref_mu = muon_ref.HostMuon({"layers.0.q_proj": params["layers.0.q_proj"]}, schedule=None)
    for t in (1, 2):
        grads = {n: (rng.standard_normal(p.shape) * 0.5).astype(np.float32) for n, p in params.items()}   # not bf16-exact
        opt.step(grads, None)
        ref_mu.step({"layers.0.q_proj": grads["layers.0.q_proj"]})
        s = adamw_ref.adamw_scalars(3e-4, 0.9, 0.95, 1e-8, t)
        for n in opt.adamw_names:
            wd = 0.0 if params[n].ndim == 1 else 0.01
            p, m, v, _ = adamw_ref.adamw_step(*st[n], grads[n].reshape(-1), s, wd)
            st[n] = [p, m, v]
    master, w = opt.master(), opt.weights()
    for n in opt.adamw_names:
        assert np.array_equal(master[n].reshape(-1), st[n][0]), n               # float32 grads: still bit-exact
        assert np.array_equal(f32_to_bf16_bits(w[n]), obf.rne_bits(master[n])), n
    a = (master["layers.0.q_proj"] - params["layers.0.q_proj"]).ravel()
    b = (ref_mu.w["layers.0.q_proj"] - params["layers.0.q_proj"]).ravel()
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 0.06
    opt.free()


def test_routing_table_matches_reference_fixture(ctx):
    t = json.load(open(os.path.join(G, "tables.json")))["routing"]
    for name, want in t.items():
        two_d = not any(k in name for k in ("_ln", "norm"))
        assert anc.default_is_muon(name, np.zeros((2, 2) if two_d else (2,))) == want, name


def test_only_adamw_or_only_muon(ctx):
    rng = np.random.default_rng(1)
    a = anc.HybridOptimizer({"embed": rng.standard_normal((64, 64)).astype(np.float32)}, ctx=ctx)
    a.step({"embed": np.ones((64, 64), np.float32)}, None)
    assert a.routing()["muon"] == [] and np.isfinite(a.weights()["embed"]).all()
    a.free()
    m = anc.HybridOptimizer({"w": rng.standard_normal((128, 128)).astype(np.float32)}, ctx=ctx)
    m.step({"w": rng.standard_normal((128, 128)).astype(np.float32)}, None)
    assert m.routing()["adamw"] == [] and np.isfinite(m.weights()["w"]).all()
    m.free()


def test_muon_zero_ns_steps_and_plain_momentum(ctx):
    """ns_steps=0 leaves the Frobenius-normalised momentum as the update (the reference's host
    newton_schulz5 with steps=0, muon.py:75); nesterov=False uses the momentum buffer itself."""
    rng = np.random.default_rng(2)
    W = (rng.standard_normal((128, 256)) * 0.02).astype(np.float32)
    g = obf.rne_f32((rng.standard_normal((128, 256)) * 1e-3).astype(np.float32))
    opt = anc.Muon({"w": W}, lr=0.02, momentum=0.9, nesterov=False, ns_steps=0, ctx=ctx)
    opt.step({"w": g}, None)
    u = obf.rne_f32(g)                                           # buf = 0*0.9 + g ; u = buf
    want = W - np.float32(0.02) * obf.rne_f32(u * muon_ref.fro_recip(u))
    got = opt.master()["w"]
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max() + 1e-9
    opt.free()


def test_dbuf_views(ctx):
    """_DBuf semantics (ancora/model/resident.py:52-94): view shares memory, at_pos offsets by rows,
    a view must not be freed."""
    a = anc.DBuf(np.arange(24, dtype=np.float32).reshape(6, 4), ctx)
    assert a.__cuda_array_interface__["shape"] == (6, 4) and a.__cuda_array_interface__["version"] == 3
    v = a.view((3, 8))
    assert v.ptr == a.ptr and v.to_numpy().shape == (3, 8)
    p = a.at_pos(2)
    assert p.ptr == a.ptr + 2 * 4 * 4
    assert a.at_pos(0) is a
    with pytest.raises(RuntimeError):
        v.free()
    assert anc.dev_ptr(a) == a.ptr and anc.dev_ptr(int(a.ptr)) == a.ptr
    a.free()


def test_bad_arguments_raise(ctx):
    with pytest.raises(anc.AncoraError):
        anc.ResidentAdamW([dict(g=0, p32=0, m=0, v=0, p16=0, numel=8, wd=0.0)], ctx=ctx)     # NULL pointers
    d = anc.DBuf.zeros((64,), np.float32, ctx)
    with pytest.raises(anc.AncoraError):
        anc.ResidentAdamW([dict(g=d, p32=d, m=d, v=d, p16=d, numel=8, wd=0.0, elem_offset=4)], ctx=ctx)  # offset % 8
    from ancora_cutile_b200 import kernels as K
    with pytest.raises(anc.AncoraError):
        K.ns_gemm_phase(0, d, None, d, 1, 100, 128, ctx=ctx)                                   # not a multiple of 128
    d.free()


def test_ring_wait_runs_out_and_context_survives(ctx):
    """A stage of the staging ring that nobody fills: the bounded wait gives up, the computing warps
    agree on it and return, status bit 0x1 is set, and the context keeps working (no trap, no hang)."""
    import ctypes as C
    from ancora_cutile_b200 import _lib as L
    ctx.sync()
    assert ctx.status() == 0
    L.check(L.lib().anc_ring_wait_selftest(ctx.handle, C.c_uint32(500)))
    assert ctx.status() == 0x1
    assert ctx.status() == 0                                       # reading clears it
    with pytest.raises(anc.AncoraError):
        L.check(L.lib().anc_ring_wait_selftest(ctx.handle, C.c_uint32(0)))
    # ordinary work still runs: one AdamW step through the ring, bit-exact against the oracle
    rng = np.random.default_rng(21)
    n = 5000
    p = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    opt = anc.AdamW({"w": p}, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, wd=0.01, ctx=ctx)
    opt.step({"w": g}, ctx.stream)
    ctx.sync()
    z = np.zeros(n, np.float32)
    want, _, _ = adamw_ref.adamw_update(p, z, z, g, adamw_ref.adamw_scalars(1e-3, 0.9, 0.95, 1e-8, 1), 0.01)
    assert np.array_equal(opt.master()["w"].reshape(-1), want)
    assert ctx.status() == 0
    opt.free()

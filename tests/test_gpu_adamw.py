"""GPU: the fused multi-tensor AdamW kernel against the CPU oracle, bit for bit.

The fp32 state (master, m, v) and the bf16 copy (RNE, and SR given the Philox stream)
must equal the oracle exactly.  Exact equality of SR output and of launch-shape
independence is this build's own gate; the reference's tests only ask rel 1e-5 and
weights()==RNE(master) (tests/optim/test_adamw.py:42-51), which are checked too."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import adamw_ref, bf16 as obf

pytestmark = pytest.mark.gpu

HP = dict(lr=3e-4, b1=0.9, b2=0.95, eps=1e-8)


def _state(rng, n):
    p = (rng.standard_normal(n) * 0.02).astype(np.float32)
    m = (rng.standard_normal(n) * 1e-4).astype(np.float32)
    v = np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32)
    g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    return p, m, v, g


def _run(ctx, specs, grad_dtype, rounding, seed, t, ranges=(None,), offsets=None):
    """specs: list of (p,m,v,g,wd).  Returns device results per tensor."""
    bufs, tensors = [], []
    for i, (p, m, v, g, wd) in enumerate(specs):
        gh = f32_to_bf16_bits(g) if grad_dtype == "bf16" else g
        b = dict(g=anc.DBuf(gh, ctx), p32=anc.DBuf(p, ctx), m=anc.DBuf(m, ctx), v=anc.DBuf(v, ctx),
                 p16=anc.DBuf.zeros(p.shape, np.uint16, ctx), numel=p.size, wd=wd)
        if offsets is not None:
            b["elem_offset"] = offsets[i]
        bufs.append(b)
        tensors.append(b)
    opt = anc.ResidentAdamW(tensors, grad_dtype=grad_dtype, rounding=rounding, seed=seed, ctx=ctx)
    for r in ranges:
        if r is not None:
            opt.set_range(*r)
        opt.step(None, t=t, **HP)
    ctx.sync()
    assert ctx.status() == 0
    out = [(b["p32"].to_numpy(), b["m"].to_numpy(), b["v"].to_numpy(), b["p16"].to_numpy()) for b in bufs]
    offs = list(opt.offsets)
    opt.free()
    for b in bufs:
        for k in ("g", "p32", "m", "v", "p16"):
            b[k].free()
    return out, offs


def _oracle(specs, grad_dtype, rounding, seed, t, offs):
    s = adamw_ref.adamw_scalars(HP["lr"], HP["b1"], HP["b2"], HP["eps"], t)
    res = []
    for (p, m, v, g, wd), off in zip(specs, offs):
        gg = obf.rne_f32(g) if grad_dtype == "bf16" else g
        res.append(adamw_ref.adamw_step(p, m, v, gg, s, wd, rounding, seed, t, off))
    return res


@pytest.mark.parametrize("grad_dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rounding", ["rne", "sr"])
def test_multi_tensor_bit_exact(ctx, grad_dtype, rounding):
    rng = np.random.default_rng(0)
    # ragged sizes: vector body + scalar tail, tiny gains, an empty tensor, a multi-chunk one
    sizes = [1024, 128, 8192 * 3 + 40, 7, 0, 64, 100003]
    wds = [0.1, 0.0, 0.1, 0.0, 0.0, 0.01, 0.1]
    specs = [(*_state(rng, n), wd) for n, wd in zip(sizes, wds)]
    got, offs = _run(ctx, specs, grad_dtype, rounding, seed=1234, t=10)
    want = _oracle(specs, grad_dtype, rounding, 1234, 10, offs)
    for i, (g_, w_) in enumerate(zip(got, want)):
        for name, a, b in zip(("p32", "m", "v", "p16"), g_, w_):
            assert np.array_equal(a.view(np.uint32) if a.dtype == np.float32 else a,
                                  b.view(np.uint32) if b.dtype == np.float32 else b), (i, name)


def test_sharded_ranges_equal_whole(ctx):
    """ZeRO-1 slices: stepping disjoint arena ranges one after another gives the same bits
    as one launch over the whole arena (the SR stream is keyed on the global index)."""
    rng = np.random.default_rng(1)
    sizes = [4096 * 5, 1024, 128, 30000]
    specs = [(*_state(rng, n), 0.1) for n in sizes]
    whole, offs = _run(ctx, specs, "bf16", "sr", seed=99, t=3)
    total = offs[-1] + sizes[-1]
    cuts = [0, 8 * 1003, 8 * 2500, 8 * 2501, (total + 7) // 8 * 8]
    parts, _ = _run(ctx, specs, "bf16", "sr", seed=99, t=3,
                    ranges=[(a, b) for a, b in zip(cuts[:-1], cuts[1:])])
    for a, b in zip(whole, parts):
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def test_unaligned_pointers_take_scalar_path(ctx):
    rng = np.random.default_rng(2)
    n = 5000
    p, m, v, g = _state(rng, n + 1)
    big = dict(g=anc.DBuf(f32_to_bf16_bits(g), ctx), p32=anc.DBuf(p, ctx), m=anc.DBuf(m, ctx),
               v=anc.DBuf(v, ctx), p16=anc.DBuf.zeros((n + 1,), np.uint16, ctx))
    t = dict(g=big["g"].slice_elems(1, n), p32=big["p32"].slice_elems(1, n), m=big["m"].slice_elems(1, n),
             v=big["v"].slice_elems(1, n), p16=big["p16"].slice_elems(1, n), numel=n, wd=0.1)
    opt = anc.ResidentAdamW([t], grad_dtype="bf16", rounding="sr", seed=5, ctx=ctx)
    opt.step(None, t=2, **HP)
    ctx.sync()
    s = adamw_ref.adamw_scalars(HP["lr"], HP["b1"], HP["b2"], HP["eps"], 2)
    pn, mn, vn, p16 = adamw_ref.adamw_step(p[1:], m[1:], v[1:], obf.rne_f32(g[1:]), s, 0.1, "sr", 5, 2, 0)
    assert np.array_equal(big["p32"].to_numpy()[1:], pn)
    assert np.array_equal(big["m"].to_numpy()[1:], mn)
    assert np.array_equal(big["v"].to_numpy()[1:], vn)
    assert np.array_equal(big["p16"].to_numpy()[1:], p16)
    assert big["p32"].to_numpy()[0] == p[0]            # the element before the view is untouched
    opt.free()
    for b in big.values():
        b.free()


def test_reference_style_test(ctx):
    """Port of tests/optim/test_adamw.py:19-53 through the host-API class."""
    rng = np.random.default_rng(0)
    lr, b1, b2, eps, wd = 0.01, 0.9, 0.999, 1e-8, 0.01
    p_w = (rng.standard_normal((256, 64)) * 0.1).astype(np.float32)
    p_n = (1.0 + rng.standard_normal(64) * 0.05).astype(np.float32)
    opt = anc.AdamW({"w": p_w.copy(), "n": p_n.copy()}, lr=lr, betas=(b1, b2), eps=eps, wd=wd,
                    no_decay=("n",), ctx=ctx)
    ref = {"w": [p_w.copy(), 0.0, 0.0, wd], "n": [p_n.copy(), 0.0, 0.0, 0.0]}
    for t in range(1, 6):
        grads = {"w": (rng.standard_normal((256, 64)) * 0.5).astype(np.float32),
                 "n": (rng.standard_normal(64) * 0.5).astype(np.float32)}
        opt.step(grads, None)
        master = opt.master()
        for name in ("w", "n"):
            p, m, v, wdi = ref[name]; g = grads[name]
            m = b1 * m + (1 - b1) * g; v = b2 * v + (1 - b2) * g * g
            mh = m / (1 - b1 ** t); vh = v / (1 - b2 ** t)
            p = p - lr * (mh / (np.sqrt(vh) + eps) + wdi * p)
            ref[name] = [p, m, v, wdi]
            e = np.abs(master[name] - p).max() / (np.abs(p).max() + 1e-9)
            assert e < 1e-5, (t, name, e)
    w16 = opt.weights()["w"]
    assert np.abs(w16 - bits_to_f32(f32_to_bf16_bits(opt.master()["w"]))).max() == 0
    opt.free()


def test_sr_is_unbiased_and_deterministic(ctx):
    """tests/kernels/_probe_sr_ops.py:41-66 semantics: fixed seed -> identical bits; the mean
    over many seeds approaches the fp32 value far better than round-to-nearest's error."""
    n = 4096
    p = np.full(n, 0.1234567, np.float32)
    z = np.zeros(n, np.float32)
    outs = []
    for seed in range(64):
        got, _ = _run(ctx, [(p, z, z, z, 0.0)], "bf16", "sr", seed=seed, t=1)
        outs.append(bits_to_f32(got[0][3]).astype(np.float64))
    again, _ = _run(ctx, [(p, z, z, z, 0.0)], "bf16", "sr", seed=63, t=1)
    assert np.array_equal(bits_to_f32(again[0][3]).astype(np.float64), outs[-1])
    master = got[0][0].astype(np.float64)
    sr_err = abs(np.mean(outs) - master.mean())
    rne_err = abs(bits_to_f32(f32_to_bf16_bits(got[0][0])).astype(np.float64).mean() - master.mean())
    assert sr_err < rne_err / 20


def test_zero_and_special_operands_bit_exact(ctx):
    """Embedding rows no token touched (g = m = v = 0 for ever), signed zeros, denormals, infinities
    and NaNs: the kernel steers zeros round the slow paths of the correctly rounded square root and
    division, and must still produce the IEEE results of the reference's statements
    (ancora/optim/adamw.py:34-37) bit for bit (NaNs compared as NaNs)."""
    rng = np.random.default_rng(77)
    n = 3 * 2048 + 37                                    # ring stages and a ragged tail
    p, m, v, g = _state(rng, n)
    m[:1500] = 0; v[:1500] = 0; g[:1500] = 0              # untouched rows
    g[1500:1600] = -0.0; m[1500:1600] = 0; v[1500:1600] = 0
    m[1600:1700] = -0.0; g[1600:1700] = 0                 # num = -0 with v > 0
    v[1700:1720] = np.inf; g[1700:1720] = 0; m[1700:1720] = 0      # 0 / inf
    v[1720:1740] = np.nan; g[1720:1740] = 0; m[1720:1740] = 0      # 0 / NaN = NaN
    g[1740:1760] = np.nan
    m[1760:1780] = np.inf
    v[1780:1800] = np.float32(1e-42)                      # denormal second moment
    g[1800:1820] = np.float32(1e-30)                      # g*g underflows to zero
    v[1800:1820] = 0; m[1800:1820] = 0
    v[-37:] = 0; m[-37:] = 0; g[-37:] = 0                 # the ragged tail (plain-load path) too
    specs = [(p, m, v, g, 0.1)]
    for grad_dtype in ("f32", "bf16"):
        got, offs = _run(ctx, specs, grad_dtype, "rne", 0, 3)
        with np.errstate(all="ignore"):
            want = _oracle(specs, grad_dtype, "rne", 0, 3, offs)
        for k in range(3):                               # p, m, v
            a, b = got[0][k], want[0][k]
            nan = np.isnan(b)
            assert np.array_equal(np.isnan(a), nan), (grad_dtype, k)
            assert np.array_equal(a[~nan].view(np.uint32), b[~nan].view(np.uint32)), (grad_dtype, k)
        fin = ~np.isnan(want[0][0])
        assert np.array_equal(got[0][3][fin], want[0][3][fin]), grad_dtype
        assert fin.sum() > n - 200 and (~fin).sum() >= 40


def test_special_operands_equal_the_reference_statements(ctx):
    """The device kernel on the fixture recorded from the reference's own statements on special
    operands (tests/golden/adamw_special.npz), float32 gradients, several copies of the 64 cases so that
    they pass through a ring stage."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "adamw_special.npz"))
    lr, b1, b2, eps, wd, t = z["hyper"]
    rep = 40                                              # 2560 elements: one full stage and a part
    tile = lambda a: np.tile(a, rep).astype(np.float32)
    p, m, v, g = tile(z["p"]), tile(z["m"]), tile(z["v"]), tile(z["g"])
    b = dict(g=anc.DBuf(g, ctx), p32=anc.DBuf(p, ctx), m=anc.DBuf(m, ctx), v=anc.DBuf(v, ctx),
             p16=anc.DBuf.zeros(p.shape, np.uint16, ctx), numel=p.size, wd=float(wd))
    opt = anc.ResidentAdamW([b], grad_dtype="f32", rounding="rne", ctx=ctx)
    opt.step(None, lr=float(lr), b1=float(b1), b2=float(b2), eps=float(eps), t=int(t))
    ctx.sync()
    assert ctx.status() == 0
    for name, buf in (("pn", b["p32"]), ("mn", b["m"]), ("vn", b["v"])):
        got, want = buf.to_numpy(), tile(z[name])
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got), nan), name
        assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)), name
    opt.free()
    for k in ("g", "p32", "m", "v", "p16"):
        b[k].free()

"""CPU: the oracle against the golden fixtures recorded from the reference's own code
(tests/golden/make_golden.py) and against published known-answer vectors."""
import json
import os

import numpy as np

from oracle import adamw_ref, bf16, muon_ref, philox, quant_ref

G = os.path.join(os.path.dirname(__file__), "golden")


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / (np.linalg.norm(b) + 1e-30))


def test_philox_known_answers():
    for ctr, key, want in philox.KNOWN_ANSWERS:
        got = philox.philox4x32_10(*ctr, *key)
        assert tuple(int(x) for x in got) == want


def test_philox_dither_layout():
    idx = np.arange(3, 203, dtype=np.uint64)
    a = philox.dither16(idx, seed=1234, step=10)
    b = philox.dither16_range(3, 200, seed=1234, step=10)
    assert np.array_equal(a, b)
    # element j of block blk: word j//2, low half for even j
    w = philox.philox4x32_10(5, 0, 10, 0, 1234, 0)
    assert int(philox.dither16(np.array([40], np.uint64), 1234, 10)[0]) == int(w[0]) & 0xFFFF
    assert int(philox.dither16(np.array([43], np.uint64), 1234, 10)[0]) == int(w[1]) >> 16
    # 64-bit seed/step/index reach the key and the counter
    assert not np.array_equal(philox.dither16_range(0, 64, 1 << 40, 1), philox.dither16_range(0, 64, 0, 1))
    assert not np.array_equal(philox.dither16_range(0, 64, 7, 1 << 33), philox.dither16_range(0, 64, 7, 0))
    assert not np.array_equal(philox.dither16_range(1 << 36, 64, 7, 1), philox.dither16_range(0, 64, 7, 1))


def test_bf16_rounding_matches_reference():
    z = np.load(os.path.join(G, "bf16.npz"))
    assert np.array_equal(bf16.rne_bits(z["x"]), z["bits"])
    assert np.array_equal(bf16.bits_f32(z["bits"]), z["back"])
    assert np.array_equal(bf16.rne_f32(z["x"]), z["bf"])
    assert bf16.rne_bits(np.array([np.nan], np.float32))[0] == 0x7FFF


def test_sr_bit_rule():
    x = np.array([1.0, -1.0, 1.00390625, 0.1, -0.1, np.inf, -np.inf, np.nan], np.float32)
    # dither 0 truncates, representable values are fixed points for every dither
    assert np.array_equal(bf16.sr_bits(x[:3], np.zeros(3)), (bf16.f32_bits(x[:3]) >> 16).astype(np.uint16))
    assert np.array_equal(bf16.sr_bits(x[:2], np.full(2, 0xFFFF)), bf16.sr_bits(x[:2], np.zeros(2)))
    lo = int(bf16.f32_bits(x[3:4])[0]) & 0xFFFF
    up = bf16.sr_bits(x[3:4], np.array([0x10000 - lo]))[0]
    dn = bf16.sr_bits(x[3:4], np.array([0x10000 - lo - 1]))[0]
    assert up == dn + 1                       # rounds up exactly when low16 + dither carries
    assert bf16.sr_bits(x[5:7], np.full(2, 0xFFFF)).tolist() == [0x7F80, 0xFF80]
    assert bf16.sr_bits(x[7:8], np.array([0xFFFF]))[0] == 0x7FFF
    # unbiased: mean over many dithers approaches the value (tests/kernels/_probe_sr_ops.py idea)
    d = np.arange(65536)
    v = np.full(65536, 0.1, np.float32)
    assert abs(bf16.bits_f32(bf16.sr_bits(v, d)).astype(np.float64).mean() - np.float64(np.float32(0.1))) < 1e-9


def test_tables_match_reference():
    t = json.load(open(os.path.join(G, "tables.json")))
    assert [list(x) for x in muon_ref.PE_SCHEDULE] == t["pe_schedule"]
    assert list(muon_ref.KELLER) == t["keller"]
    assert [list(muon_ref.coef_at(muon_ref.PE_SCHEDULE, k)) for k in range(8)] == t["coef_at_pe"]
    assert [list(muon_ref.coef_at(None, k)) for k in range(3)] == t["coef_at_none"]


def test_ns_fp32_keller_golden():
    z = np.load(os.path.join(G, "ns_keller.npz"))
    for i in range(3):
        out = muon_ref.ns_fp32(z[f"in{i}"], 5, None)
        assert out.shape == z[f"out{i}"].shape
        assert _rel(out, z[f"out{i}"]) < 2e-5     # BLAS summation order may differ between hosts


def test_ns_fp32_polar_express_golden():
    z = np.load(os.path.join(G, "ns_pe.npz"))
    for i in range(2):
        assert _rel(muon_ref.ns_fp32(z[f"in{i}"], 5, muon_ref.PE_SCHEDULE), z[f"out{i}"]) < 2e-5
        assert _rel(muon_ref.ns_fp32(z[f"in{i}"], 7, muon_ref.PE_SCHEDULE), z[f"out{i}_n7"]) < 2e-5


def test_host_muon_golden():
    z = np.load(os.path.join(G, "host_muon.npz"))
    names = ("tall", "wide")
    opt = muon_ref.HostMuon({k: z[f"p_{k}"] for k in names})
    for t in range(3):
        opt.step({k: z[f"g{t}_{k}"] for k in names})
    for k in names:
        assert _rel(opt.w[k], z[f"master_{k}"]) < 1e-6
        assert np.array_equal(opt.buf[k], z[f"buf_{k}"])          # momentum is BLAS-free: exact
        w = opt.weights()[k]
        assert np.mean(w != z[f"weights_{k}"]) < 1e-3


def test_adamw_oracle_vs_reference_test_formula():
    """The reference's own check (tests/optim/test_adamw.py:19-51): 5 steps, two tensors,
    kernel-order result within rel 1e-5 of the divide-form numpy; weights == RNE(master)."""
    rng = np.random.default_rng(0)
    lr, b1, b2, eps, wd = 0.01, 0.9, 0.999, 1e-8, 0.01
    P = {"w": (rng.standard_normal((256, 64)) * 0.1).astype(np.float32),
         "n": (1.0 + rng.standard_normal(64) * 0.05).astype(np.float32)}
    wds = {"w": wd, "n": 0.0}
    st = {k: [v.copy(), np.zeros_like(v), np.zeros_like(v)] for k, v in P.items()}
    ref = {k: [v.copy(), 0.0, 0.0] for k, v in P.items()}
    for t in range(1, 6):
        g = {"w": (rng.standard_normal((256, 64)) * 0.5).astype(np.float32),
             "n": (rng.standard_normal(64) * 0.5).astype(np.float32)}
        s = adamw_ref.adamw_scalars(lr, b1, b2, eps, t)
        for k in P:
            p, m, v, p16 = adamw_ref.adamw_step(*st[k], g[k], s, wds[k])
            st[k] = [p, m, v]
            ref[k] = list(adamw_ref.adamw_reference_test_form(*ref[k], g[k], lr, b1, b2, eps, wds[k], t))
            e = np.abs(p - ref[k][0]).max() / (np.abs(ref[k][0]).max() + 1e-9)
            assert e < 1e-5
            assert np.array_equal(p16, bf16.rne_bits(p))


def test_adamw_oracle_equals_the_reference_kernel_statements_bit_for_bit():
    """adamw.npz holds the outputs of the reference kernel's own four arithmetic statements
    (ancora/optim/adamw.py:34-37), read from its source and executed on float32 numpy arrays by
    tests/golden/make_golden.py.  The oracle must reproduce them exactly, so its operation order
    is pinned to the reference's text."""
    z = np.load(os.path.join(G, "adamw.npz"))
    assert [s.split("=")[0].strip() for s in z["statements"]] == ["mn", "vn", "upd", "pn"]
    lr, b1, b2, eps, wd, t = z["hyper"]
    s = adamw_ref.adamw_scalars(lr, b1, b2, eps, int(t))
    with np.errstate(all="ignore"):
        pn, mn, vn, p16 = adamw_ref.adamw_step(z["p"], z["m"], z["v"], z["g"], s, wd, "rne")
    for name, got in (("mn", mn), ("vn", vn), ("pn", pn)):
        assert np.array_equal(got.view(np.uint32), z[name].view(np.uint32)), name
    assert np.array_equal(p16, z["p16"])


def test_adamw_oracle_on_special_operands_equals_the_reference_statements():
    """adamw_special.npz: the same four statements of the reference on rows no token touched
    (g = m = v = 0), signed zeros, denormal / infinite / NaN moments and gradients.  Finite results and
    zeros equal bit for bit (the sign of a zero included), NaNs are NaNs in the same places."""
    z = np.load(os.path.join(G, "adamw_special.npz"))
    lr, b1, b2, eps, wd, t = z["hyper"]
    s = adamw_ref.adamw_scalars(lr, b1, b2, eps, int(t))
    with np.errstate(all="ignore"):
        pn, mn, vn, _ = adamw_ref.adamw_step(z["p"], z["m"], z["v"], z["g"], s, wd, "rne")
    for name, got in (("mn", mn), ("vn", vn), ("pn", pn)):
        want = z[name]
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got), nan), name
        assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)), name
    assert np.isnan(z["pn"]).sum() == 8 and np.isinf(z["vn"]).sum() == 4 and np.isinf(z["pn"]).sum() == 4   # the cases are there
    assert np.array_equal(z["pn"][:8].view(np.uint32), (z["p"][:8] - np.float32(lr) * (np.float32(wd) * z["p"][:8])).view(np.uint32))


def test_adamw_scalars_definition():
    s = adamw_ref.adamw_scalars(3e-4, 0.9, 0.95, 1e-8, 10)
    assert s.omb1 == np.float32(1.0) - np.float32(0.9)          # float32 subtraction, adamw.py:34
    assert s.omb1 != np.float32(1 - 0.9)                        # differs from the double form by 1 ulp
    assert s.ibc1 == np.float32(1.0 / (1.0 - 0.9 ** 10))


def test_bf16_chain_model_within_tolerance():
    rng = np.random.default_rng(3)
    for shp in [(128, 384), (256, 256)]:
        g = bf16.rne_bits((rng.standard_normal(shp) * 1e-3).astype(np.float32))
        want = muon_ref.ns_fp32(bf16.bits_f32(g), 5, muon_ref.PE_SCHEDULE)
        got = bf16.bits_f32(muon_ref.ns_bf16_chain(g, 5, muon_ref.PE_SCHEDULE))
        assert _rel(got, want) < 2e-2


def test_oracle_quant_decodes_within_e4m3_step():
    rng = np.random.default_rng(0)
    w = bf16.rne_bits((rng.standard_normal((128, 96)) * np.exp(rng.uniform(-8, 2, (1, 96)))).astype(np.float32))
    q, byte = quant_ref.quant_mxfp8_w(w)
    back = quant_ref.dequant_mxfp8_w(q, byte)
    x = bf16.bits_f32(w).astype(np.float64)
    blockmax = np.abs(x).reshape(4, 32, 96).max(axis=1).repeat(32, axis=0)
    assert np.all(np.abs(back - x) <= blockmax * 2.0 ** -4 + 1e-30)       # 3 mantissa bits, block-relative
    assert np.all(q[np.abs(x) == blockmax] != 0)


def test_polar_express_orthogonalises_better_than_keller_in_five_steps():
    """Host-only property the reference checks in tests/kernels/_probe_polar_express.py: on
    matrices with spread singular values, 5 Polar-Express iterations leave a smaller
    orthogonality error than 5 Keller iterations, and a sixth PE step (last triple repeated,
    muon_ns.py:38-42) does not make it worse."""
    from oracle import muon_ref
    rng = np.random.default_rng(0)
    for M, N in ((128, 128), (128, 384)):
        W = (rng.standard_normal((M, N)) @ np.diag(rng.uniform(0.1, 3.0, N))).astype(np.float32)

        def err(Y):
            return float(np.linalg.norm(Y @ Y.T - np.eye(M, dtype=Y.dtype)) / np.sqrt(M))

        k5 = err(muon_ref.ns_fp32(W, 5, None))
        p5 = err(muon_ref.ns_fp32(W, 5, muon_ref.PE_SCHEDULE))
        p6 = err(muon_ref.ns_fp32(W, 6, muon_ref.PE_SCHEDULE))
        assert p5 < k5, (M, N, p5, k5)
        assert p6 <= p5 * 1.05, (M, N, p6, p5)


def test_e4m3_oracle_against_the_reference_host_helpers():
    """oracle/quant_ref.py against fixtures recorded from ancora/kernels/quant.py's host code: the
    decode table bit for bit; the rounding equal to f32_to_e4m3 wherever the input is not an exact
    tie (the host helper sends ties to the smaller magnitude, the device conversion the kernels use
    is round-to-nearest-even, which the oracle follows: at a tie it must pick the even one of the
    two neighbours); the block dequantisation equal to dequantize_rowblock."""
    from oracle import quant_ref
    g = np.load(os.path.join(G, "e4m3.npz"))
    tab = quant_ref.e4m3_table()
    assert np.array_equal(np.nan_to_num(tab.astype(np.float32), nan=-7.0), np.nan_to_num(g["table"], nan=-7.0))
    x, ref = g["x"], g["bytes"]
    got = quant_ref._e4m3_rne(np.clip(x, -448.0, 448.0))          # the host helper saturates at 448
    pos = tab[:127]
    ax = np.minimum(np.abs(x).astype(np.float64), 448.0)
    hi = np.clip(np.searchsorted(pos, ax), 1, 126)
    lo = hi - 1
    tie = (ax - pos[lo]) == (pos[hi] - ax)
    assert tie.sum() > 100 and (~tie).sum() > 1000
    same = (got & 0x7F) == (ref & 0x7F)
    assert same[~tie].all()
    assert np.array_equal(got & 0x80, ref & 0x80)                  # signs, signed zero included
    even = np.where(lo % 2 == 0, lo, hi)
    assert np.array_equal((got & 0x7F)[tie], even[tie].astype(np.uint8))
    # dequantisation: the reference lays blocks along the last axis, the weight form along axis 0
    want = g["dequant"]
    mine = quant_ref.dequant_mxfp8_w(np.ascontiguousarray(g["fp8"].T), np.ascontiguousarray(g["scale"].T)).T
    assert np.array_equal(mine.astype(np.float32), want)

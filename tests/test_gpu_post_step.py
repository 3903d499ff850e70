"""GPU: post-step consumers fused into the Muon update -- the MXFP8 re-quantisation and the
transposed bf16 copy -- against the oracle, byte for byte, and unchanged main outputs."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import bf16 as obf, quant_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which", ["all", "transposed_only"])
@pytest.mark.parametrize("shape", [(128, 256), (256, 128), (128, 128)])
def test_fused_outputs_match_oracle_and_main_outputs_unchanged(ctx, shape, which):
    K, N = shape
    rng = np.random.default_rng(1)
    W = (rng.standard_normal(shape) * np.exp(rng.uniform(-6, 1, (1, N)))).astype(np.float32)
    g = f32_to_bf16_bits((rng.standard_normal(shape) * 1e-3).astype(np.float32))

    def run(extras):
        w = dict(buf=anc.DBuf.zeros(shape, np.float32, ctx), p32=anc.DBuf(W, ctx),
                 p16=anc.DBuf(f32_to_bf16_bits(W), ctx), G=anc.DBuf(g, ctx), K=K, N=N)
        if extras:
            w.update(fp8_t=anc.DBuf.zeros((N, K), np.uint8, ctx),
                     fp8_scale_t=anc.DBuf.zeros((N, K // 32), np.uint8, ctx))
        if extras and which == "all":
            w.update(fp8=anc.DBuf.zeros(shape, np.uint8, ctx), fp8_scale=anc.DBuf.zeros((K // 32, N), np.uint8, ctx),
                     p16_t=anc.DBuf.zeros((N, K), np.uint16, ctx))
        bp = anc.BatchedProjMuon([w], grad_dtype="bf16", schedule=anc.PE_SCHEDULE, ctx=ctx)
        for _ in range(2):
            bp.step(ctx.stream, 0.02)
        ctx.sync()
        assert ctx.status() == 0
        out = {k: w[k].to_numpy() for k in w if isinstance(w[k], anc.DBuf)}
        bp.free()
        for k in list(w):
            if isinstance(w[k], anc.DBuf):
                w[k].free()
        return out

    plain, fused = run(False), run(True)
    for k in ("p32", "p16", "buf"):
        assert np.array_equal(plain[k], fused[k]), k
    assert np.array_equal(fused["p16"], f32_to_bf16_bits(fused["p32"]))
    q_t, byte_t = quant_ref.quant_mxfp8_w_cm(fused["p16"])
    assert np.array_equal(fused["fp8_scale_t"], byte_t)
    assert np.array_equal(fused["fp8_t"], q_t)
    if which == "all":
        assert np.array_equal(fused["p16_t"], fused["p16"].T)
        q, byte = quant_ref.quant_mxfp8_w(fused["p16"])
        assert np.array_equal(fused["fp8_scale"], byte)
        assert np.array_equal(fused["fp8"], q)

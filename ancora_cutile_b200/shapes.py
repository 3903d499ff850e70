"""Parameter shape lists of the two benchmark model families (synthetic state only).

Shapes follow the reference's (in, out) weight convention (ancora/model/load_qwen3.py:38-44,
ancora/model/qwen3_layer.py:105-109): q (H, Hq*D), k/v (H, Hkv*D), o (Hq*D, H),
gate/up (H, I), down (I, H).  Names follow its params() scheme
(ancora/model/qwen3_model.py:41-46, moe_model.py:51-60) so ``default_is_muon`` routes them
as in the reference.
"""
import numpy as np


def qwen3_0_6b_shapes(n_layers=28, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, ffn=3072,
                      vocab=151936):
    s = {"embed": (vocab, hidden)}
    for l in range(n_layers):
        p = f"layers.{l}."
        s[p + "input_ln"] = (hidden,)
        s[p + "q_proj"] = (hidden, q_heads * head_dim)
        s[p + "k_proj"] = (hidden, kv_heads * head_dim)
        s[p + "v_proj"] = (hidden, kv_heads * head_dim)
        s[p + "q_norm"] = (head_dim,)
        s[p + "k_norm"] = (head_dim,)
        s[p + "o_proj"] = (q_heads * head_dim, hidden)
        s[p + "post_ln"] = (hidden,)
        s[p + "gate_proj"] = (hidden, ffn)
        s[p + "up_proj"] = (hidden, ffn)
        s[p + "down_proj"] = (ffn, hidden)
    s["final_norm"] = (hidden,)
    return s


def moe_family_shapes(n_layers=24, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, ffn=3072,
                      experts=16, expert_ffn=768, vocab=151936):
    """Alternating dense / MoE layers; each expert has gate/up (H, Ie) and down (Ie, H)."""
    s = {"embed": (vocab, hidden)}
    for l in range(n_layers):
        p = f"layers.{l}."
        s[p + "input_ln"] = (hidden,)
        s[p + "q_proj"] = (hidden, q_heads * head_dim)
        s[p + "k_proj"] = (hidden, kv_heads * head_dim)
        s[p + "v_proj"] = (hidden, kv_heads * head_dim)
        s[p + "q_norm"] = (head_dim,)
        s[p + "k_norm"] = (head_dim,)
        s[p + "o_proj"] = (q_heads * head_dim, hidden)
        s[p + "post_ln"] = (hidden,)
        if l % 2 == 0:
            s[p + "gate_proj"] = (hidden, ffn)
            s[p + "up_proj"] = (hidden, ffn)
            s[p + "down_proj"] = (ffn, hidden)
        else:
            s[p + "router"] = (hidden, experts)            # 2-D but not tileable: AdamW (HybridOptimizer's fallback)
            for e in range(experts):
                q = p + f"experts.{e}."
                s[q + "gate_proj"] = (hidden, expert_ffn)
                s[q + "up_proj"] = (hidden, expert_ffn)
                s[q + "down_proj"] = (expert_ffn, hidden)
    s["final_norm"] = (hidden,)
    return s


def synthetic_params(shapes, seed=0, std=0.02):
    """fp32 masters ~ N(0, std^2) (gains ~ 1 + N(0, std^2)), one generator stream per tensor
    in registration order."""
    rng = np.random.default_rng(seed)
    out = {}
    for n, shp in shapes.items():
        x = rng.standard_normal(shp, dtype=np.float32) * np.float32(std)
        if len(shp) == 1:
            x += np.float32(1.0)
        out[n] = x
    return out


def synthetic_grads_bf16(shapes, seed=1, std=1e-3, out=None):
    """bf16-bit gradients ~ N(0, std^2); fills ``out[name]`` in place when given."""
    from .bf16 import f32_to_bf16_bits
    rng = np.random.default_rng(seed)
    res = {}
    for n, shp in shapes.items():
        g = f32_to_bf16_bits(rng.standard_normal(shp, dtype=np.float32) * np.float32(std)).reshape(shp)
        if out is not None:
            np.copyto(out[n], g)
            res[n] = out[n]
        else:
            res[n] = g
    return res


def count(shapes):
    return int(sum(int(np.prod(s, dtype=np.int64)) for s in shapes.values()))

"""Times of the HBM-bound sweeps (AdamW, Muon momentum and update) per shape group.

    python -m ancora_cutile_b200.profile_sweeps [--layers 28] [--steps 5]

Builds the Muon state of a Qwen3-0.6B-shaped model (seven projections per layer, registered in layer
order, in four arenas) and an AdamW arena of the embedding's size, filled with seeded values, and runs
whole optimizer steps queued back to back the way ``bench.py`` does.  Prints, per shape group, the
CUDA-event time of the momentum and the update launch and the algorithmic bandwidth (12 B per element
each), once with every group run and synchronised on its own and once as the sum over whole steps, and the
AdamW launch (28 B per element).  Use it to compare builds of the sweeps on one box; ``bench.py`` gives the
numbers inside the full step.
"""
import argparse

import numpy as np

from . import muon_ns
from .adamw import ResidentAdamW
from .buffers import DBuf, Event, get_context
from .muon import MuonPlan

PROJECTIONS = [(1024, 2048), (1024, 1024), (1024, 1024), (2048, 1024), (1024, 3072), (1024, 3072), (3072, 1024)]


def _arena(ctx, rng, total, dtype, scale, positive=False):
    a = DBuf.empty((total,), dtype, ctx)
    blk = 1 << 24
    for s in range(0, total, blk):
        n = min(blk, total - s)
        x = (rng.standard_normal(n) * scale).astype(np.float32)
        if positive:
            x = np.abs(x)
        if dtype == np.uint16:
            x = (x.view(np.uint32) >> 16).astype(np.uint16)
        a.slice_elems(s, n).upload(x)
    return a


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--adamw-elems", type=int, default=155_648_000)
    ap.add_argument("--adamw-zeros", action="store_true",
                    help="AdamW gradients and moments all zero (embedding rows no token touched)")
    args = ap.parse_args()
    ctx = get_context()
    rng = np.random.default_rng(0)
    shapes = PROJECTIONS * args.layers
    total = sum(k * n for k, n in shapes)
    buf, g = _arena(ctx, rng, total, np.float32, 1e-3), _arena(ctx, rng, total, np.uint16, 1e-3)
    p32, p16 = _arena(ctx, rng, total, np.float32, 0.02), _arena(ctx, rng, total, np.uint16, 0.02)
    ws, off = [], 0
    for k, n in shapes:
        ws.append(dict(buf=buf.slice_elems(off, k * n), G=g.slice_elems(off, k * n), p32=p32.slice_elems(off, k * n),
                       p16=p16.slice_elems(off, k * n), K=k, N=n))
        off += k * n
    plan = MuonPlan(ws, grad_dtype="bf16", ctx=ctx)
    plan.set_timing(True)
    sched = muon_ns.PE_SCHEDULE
    na = args.adamw_elems // 2048 * 2048
    # seeded state, not zeros: IEEE division and square root take their slow paths on zero operands
    z = 0.0 if args.adamw_zeros else 1.0
    aw = ResidentAdamW([dict(g=_arena(ctx, rng, na, np.uint16, 1e-3 * z), p32=_arena(ctx, rng, na, np.float32, 0.02),
                             m=_arena(ctx, rng, na, np.float32, 1e-4 * z), v=_arena(ctx, rng, na, np.float32, 1e-6 * z, True),
                             p16=DBuf.zeros((na,), np.uint16, ctx), numel=na, wd=0.1)],
                       grad_dtype="bf16", rounding="sr", seed=1, ctx=ctx)

    # every group on its own
    ng = plan.num_groups()
    acc = {}
    for it in range(args.steps + 1):
        for gi in range(ng):
            cnt, _, M, N = plan.group_info(gi)
            plan.step_range(gi, 0, cnt, None, 0.02, 0.95, True, 5, sched)
            ctx.sync()
            t = plan.last_timing()
            if it:
                a = acc.setdefault(gi, [0.0, 0.0, cnt * M * N * 12 / 1e6, (cnt, M, N)])
                a[0] += t["momentum_ms"]
                a[1] += t["update_ms"]
    for gi, a in acc.items():
        m, u = a[0] / args.steps, a[1] / args.steps
        print(f"group {a[3]}: momentum {m:.4f} ms ({a[2] / m:.0f} GB/s)  update {u:.4f} ms ({a[2] / u:.0f} GB/s)")

    # whole steps queued back to back: AdamW, then the groups by descending size
    order = sorted(range(ng), key=lambda gi: -plan.group_info(gi)[0] * plan.group_info(gi)[2] * plan.group_info(gi)[3])
    e0, e1 = Event(), Event()
    spans = []

    def step(timed):
        if timed:
            a, b = Event(), Event()
            a.record(ctx.stream)
        aw.step(None)
        if timed:
            b.record(ctx.stream)
            spans.append((a, b))
        for gi in order:
            plan.step_range(gi, 0, plan.group_info(gi)[0], None, 0.02, 0.95, True, 5, sched)

    step(False)
    ctx.sync()
    plan.last_timing()
    e0.record(ctx.stream)
    for _ in range(args.steps):
        step(True)
    e1.record(ctx.stream)
    ctx.sync()
    t = plan.last_timing()
    k = args.steps
    aw_ms = sum(a.elapsed_ms(b) for a, b in spans) / k
    mb = total * 12 / 1e6
    print(f"queued back to back, per step: AdamW {aw_ms:.4f} ms ({na * 28 / 1e6 / aw_ms:.0f} GB/s)  "
          f"momentum {t['momentum_ms'] / k:.4f} ms ({mb / (t['momentum_ms'] / k):.0f} GB/s)  "
          f"update {t['update_ms'] / k:.4f} ms ({mb / (t['update_ms'] / k):.0f} GB/s)  "
          f"chains {t['ns_ms'] / k:.3f} ms  step {e0.elapsed_ms(e1) / k:.3f} ms  status {ctx.status()}")


if __name__ == "__main__":
    main()

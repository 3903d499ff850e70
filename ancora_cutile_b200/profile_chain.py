"""Per-role stall accounting of the Newton-Schulz chain kernel.

    python -m ancora_cutile_b200.build --profile
    python -m ancora_cutile_b200.profile_chain [E,M,N ...]

The profile build (-DANC_CHAIN_PROFILE) makes every role of ``ns_chain_kernel`` add the cycles
it spends in each of its waits to a per-CTA row of a device array; this script runs the chain
on seeded matrices of the given shapes (default: the benchmark's shape groups, whole and cut to
one rank's share at 8 GPUs) and prints, per role, where its time went.  The numbers come from
``clock64`` inside the kernel, so the profile build runs a few per cent slower than the
library proper: use them for shares, and ``bench.py`` for times.
"""
import ctypes as C
import os
import sys

import numpy as np

from . import _lib as L

L.LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libancora_b200_prof.so")

from . import muon_ns                                     # noqa: E402
from .bf16 import f32_to_bf16_bits                         # noqa: E402
from .buffers import DBuf, Event, get_context              # noqa: E402

ROLES = {0: ("producer", ["issue", "tile wait", "stage wait"]),
         1: ("mma", ["issue", "tile wait", "accumulator wait", "operand wait"]),
         2: ("epilogue", ["tile wait + tail", "operand loads", "accumulator wait", "vote + fence",
                          "tmem load 1", "combine + store 1", "tmem load 2", "combine + store 2"]),
         3: ("signal", ["other", "tile wait", "epilogue wait", "release"]),
         4: ("scheduler", ["publish", "slot wait", "claim + decode", "dependency wait"])}
N_CTAS = 296


def run(E, M, N, steps=5, reps=3):
    ctx = get_context()
    prof = L.lib().anc_debug_chain_prof
    prof.restype = C.c_int
    rng = np.random.default_rng(0)
    Xb = f32_to_bf16_bits((rng.standard_normal((E * M, N)) * 1e-3).astype(np.float32))
    Z = lambda *s: DBuf.zeros(s, np.uint16, ctx)
    gX, gA, gB, gBX = DBuf(Xb, ctx), Z(E * M, M), Z(E * M, M), Z(E * M, N)
    gr = DBuf.zeros((E, 1), np.float32, ctx)
    buf = (C.c_ulonglong * (N_CTAS * 40))()
    e0, e1 = Event(), Event()
    for _ in range(reps):
        gX.upload(Xb)
        ctx.sync()
        prof(buf, N_CTAS)                                  # clears the counters
        e0.record(ctx.stream)
        muon_ns.newton_schulz_resident_e(gX, gA, None, gB, gBX, gr, E, M, N, ctx.stream, steps=steps,
                                         schedule=muon_ns.PE_SCHEDULE)
        e1.record(ctx.stream)
        ctx.sync()
    ms = e0.elapsed_ms(e1)
    prof(buf, N_CTAS)
    a = np.array(buf[:], dtype=np.float64).reshape(N_CTAS, 5, 8)
    nb = M // 256
    executed = E * steps * ((nb + 1) / (2 * nb) * (2.0 * M * M * N + 2.0 * M ** 3) + 2.0 * M * M * N)
    print(f"E={E} M={M} N={N}: {ms:.3f} ms, {executed / ms / 1e9:.0f} TFLOP/s executed, status {ctx.status()}")
    for role, (name, labels) in ROLES.items():
        rows = a[:, role, :]
        rows = rows[rows.sum(1) > 0]
        if not len(rows):
            continue
        tot = rows.sum(1).mean()
        parts = ", ".join(f"{l} {rows[:, k].mean() / tot * 100:.0f}%" for k, l in enumerate(labels)
                          if rows[:, k].mean() / tot > 0.005)
        print(f"   {name:9s} ({len(rows)} CTAs, {tot / 1e3:.0f} kclk): {parts}")
    for g in (gX, gA, gB, gBX, gr):
        g.free()


def main(argv):
    shapes = [tuple(int(x) for x in a.split(",")) for a in argv] or \
        [(84, 1024, 3072), (56, 1024, 2048), (56, 1024, 1024), (11, 1024, 3072), (7, 1024, 2048), (7, 1024, 1024),
         (72, 768, 1024)]
    for E, M, N in shapes:
        run(E, M, N)


if __name__ == "__main__":
    main(sys.argv[1:])

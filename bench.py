#!/usr/bin/env python
"""Benchmark of the hybrid Muon + AdamW optimizer step on Qwen3-0.6B shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload qwen3|moe]

One "step" = one full optimizer step over all 596 M parameters (196 Muon matrices, the tied
embedding and 113 gain vectors under AdamW), synthetic seeded state, bf16 gradients,
Polar-Express Newton-Schulz (5 iterations), stochastic-rounded bf16 AdamW output.
With N > 1 (launched by torch.distributed.run, one rank per GPU) the step is ZeRO-1 sharded
and ends with the NCCL all-gather of the updated bf16 parameters.

Prints ONE JSON line on rank 0.  `value` is parameters updated per second over the whole job
with all inputs resident in HBM; `e2e` is the same through HybridOptimizer.step with host
gradients (page-locked) copied in and the updated bf16 weights copied out inside the timed
region.  `--impl reference` times the reference's numpy formulation (the CPU oracle port) on
the host cores over a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

# The CPU arm uses every core this process may run on.  Launchers such as torch.distributed.run
# export OMP_NUM_THREADS=1 to their children, which would cut the BLAS of the CPU arm to one
# thread; the thread counts are therefore set here, before numpy loads its BLAS.
if "reference" in sys.argv[1:] or int(os.environ.get("WORLD_SIZE", "1")) == 1:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(len(os.sched_getaffinity(0)))

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ADAMW_KW = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1)
MUON_KW = dict(lr=0.02, momentum=0.95, nesterov=True, ns_steps=5)
SEED_SR = 1234
# ncu dram__bytes_read.sum + dram__bytes_write.sum of the Newton-Schulz GEMM kernel divided by its
# algorithmic bytes (operands once, outputs once), and the capture it comes from
GEMM_TRAFFIC_RATIO = 1.00
GEMM_TRAFFIC_SOURCE = ("ns_chain_kernel, the three full Qwen3-0.6B shape groups (84/56/56 matrices), 1-pass capture: "
                       "11.42 / 5.84 / 4.08 GB against 11.45 / 5.87 / 4.11 GB algorithmic")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), src="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake"}

    def __init__(self, device):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.th = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def start(self):
        if self.nv:
            self.th.start()

    def stop(self):
        self._stop.set()
        if self.nv and self.th.is_alive():
            self.th.join(1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def workload_shapes(name, layers=None, vocab=None):
    """layers / vocab shrink the model for profiler captures; a run that sets them is not
    the benchmark configuration and says so in config.workload."""
    from ancora_cutile_b200 import shapes
    kw = {}
    if layers:
        kw["n_layers"] = layers
    if vocab:
        kw["vocab"] = vocab
    tag = f" REDUCED for profiling: {kw}" if kw else ""
    if name == "qwen3":
        return shapes.qwen3_0_6b_shapes(**kw), "qwen3-0.6b hybrid optimizer step (28 layers, d=1024, ffn=3072, vocab=151936)" + tag
    return shapes.moe_family_shapes(**kw), "moe-family hybrid optimizer step (24 layers, 16x(768x1024) experts per MoE layer)" + tag


def route(shp):
    from ancora_cutile_b200.hybrid import muon_names_for
    return muon_names_for(shp)


# ------------------------------------------------------------------ CPU arm
def cpu_arm(shp, muon_names, total_params, steps, warmup, layers):
    """Times the reference's host optimizer step on this machine's cores.

    Muon: the reference's own host class (ancora/optim/muon.py:287-318, fp32 Newton-Schulz through
    BLAS) loaded from oracle/_ref when that was built, else the numpy port in oracle/muon_ref.py.
    AdamW: the reference has no host AdamW class; its kernel's four statements
    (ancora/optim/adamw.py:34-37) plus the round-to-nearest bf16 cast (:41) are timed through
    oracle/adamw_ref.py, which equals those statements bit for bit.  The Philox stochastic-rounding
    pass this build adds is timed separately and is NOT part of the reference's figure.

    A step covers the Muon matrices of the first `layers` layers and the same fraction of the
    AdamW elements, i.e. a sample with the workload's own composition: the rate in params/s is
    measured, not extrapolated; only ms_per_step of the whole workload is derived from it.
    """
    from oracle import adamw_ref, bf16 as obf, build_ref, muon_ref, philox
    n_layers = 1 + max(int(n.split(".")[1]) for n in muon_names)
    layers = min(layers, n_layers)
    frac = layers / n_layers
    rng = np.random.default_rng(0)
    sel = [n for n in muon_names if int(n.split(".")[1]) < layers]
    P = {n: (rng.standard_normal(shp[n], dtype=np.float32) * np.float32(0.02)) for n in sel}
    G = {n: (rng.standard_normal(shp[n], dtype=np.float32) * np.float32(1e-3)) for n in sel}
    ref, why_not = build_ref.load()
    if ref is not None:
        opt = ref[0](P, lr=MUON_KW["lr"], momentum=MUON_KW["momentum"], nesterov=True, ns_steps=MUON_KW["ns_steps"])
        kind, muon_src = "reference", "the reference's host Muon class (oracle/_ref, built from the checkout)"
    else:
        opt = muon_ref.HostMuon(P, lr=MUON_KW["lr"], momentum=MUON_KW["momentum"], nesterov=True,
                                ns_steps=MUON_KW["ns_steps"], schedule=muon_ref.PE_SCHEDULE)
        kind, muon_src = "port", f"numpy port of the reference's host Muon ({why_not})"
    a_total = sum(int(np.prod(s)) for k, s in shp.items() if k not in set(muon_names))
    n = max(64, int(a_total * frac) // 64 * 64)
    st = {"p": rng.standard_normal(n, dtype=np.float32) * np.float32(0.02),
          "m": rng.standard_normal(n, dtype=np.float32) * np.float32(1e-4),
          "v": np.abs(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-6)), "t": 0}
    g = obf.rne_f32(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3))
    sample_params = sum(int(np.prod(shp[k])) for k in sel) + n

    def step():
        t0 = time.perf_counter()
        opt.step(G)
        t1 = time.perf_counter()
        st["t"] += 1
        s = adamw_ref.adamw_scalars(ADAMW_KW["lr"], *ADAMW_KW["betas"], ADAMW_KW["eps"], st["t"])
        st["p"], st["m"], st["v"] = adamw_ref.adamw_update(st["p"], st["m"], st["v"], g, s, ADAMW_KW["wd"])
        obf.rne_bits(st["p"])
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    for _ in range(warmup):
        step()
    tm = ta = 0.0
    for _ in range(steps):
        a, b = step()
        tm += a
        ta += b
    t0 = time.perf_counter()
    obf.sr_bits(st["p"], philox.dither16_range(0, n, SEED_SR, 1))
    sr_s = time.perf_counter() - t0
    per_step = (tm + ta) / steps
    threads = len(os.sched_getaffinity(0))
    rate = sample_params / per_step
    return {"value": rate, "unit": "params/s", "cores": threads, "kind": kind,
            "ms_per_step": total_params / rate * 1e3, "extrapolated": frac < 1.0, "sample_fraction": frac,
            "sample_params": sample_params, "sample_ms_per_step": per_step * 1e3,
            "muon_ms": tm / steps * 1e3, "adamw_ms": ta / steps * 1e3,
            "philox_sr_pass_ms_not_included": sr_s * 1e3,
            "blas_threads_env": os.environ.get("OMP_NUM_THREADS"),
            "sample": (f"{muon_src}: {len(sel)} matrices of {layers}/{n_layers} layers; AdamW statements + RNE cast "
                       f"on {n} elements ({frac:.3f} of the AdamW set): the workload's composition, rate measured on "
                       f"the sample; {steps} step(s) after {warmup} warm-up, numpy {np.__version__}")}


def grad_reduce_scatter_leg(eng, pin, rank, world, ctx):
    """Rank r's local gradient is bf16(base * (1 + r/16)) for the synthetic base gradient, so every
    rank can compute the exact sum over ranks for the elements it owns."""
    from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
    base = {n: v.copy() for n, v in pin.items()}
    scale = lambda r: np.float32(1.0 + r / 16.0)
    CH = 1 << 24

    def local(bits, r):
        return f32_to_bf16_bits(bits_to_f32(bits) * scale(r))

    for n, v in pin.items():                          # this rank's local gradients, in the staging views
        flat, b = v.reshape(-1), base[n].reshape(-1)
        for lo in range(0, flat.size, CH):
            flat[lo:lo + CH] = local(b[lo:lo + CH], rank)
    eng.enable_grad_accumulation()
    digests, worst, checked, ms = [], 0.0, 0, 0.0
    e0, e1 = Event_pair()
    for rep in range(2):
        eng.upload_full_grads(pin, ctx.stream)
        e0.record(ctx.stream)
        eng.finalize_grads(ctx.stream, rounding="rne", reduce=True)
        e1.record(ctx.stream)
        ctx.sync()
        ms = e0.elapsed_ms(e1)
        import hashlib
        h = hashlib.blake2b(digest_size=16)
        for n in pin:
            lo, hi = eng.owned_range(n)
            if hi <= lo:
                continue
            got = eng.grad_view(n).to_numpy().reshape(-1)[lo:hi]
            h.update(got.tobytes())
            if rep == 0:
                b = base[n].reshape(-1)[lo:hi]
                for c in range(0, b.size, CH):
                    want = np.zeros(min(CH, b.size - c), np.float64)
                    for r in range(world):
                        want += bits_to_f32(local(b[c:c + CH], r)).astype(np.float64)
                    want /= world
                    g = bits_to_f32(got[c:c + CH]).astype(np.float64)
                    den = np.maximum(np.abs(want), 1e-30)
                    worst = max(worst, float(np.max(np.abs(g - want) / den)))
                    checked += want.size
        digests.append(h.hexdigest())
    for n, v in pin.items():                          # put the base gradient back
        np.copyto(v, base[n])
    return {"max_rel_err": worst, "repeatable_bits": digests[0] == digests[1], "elements_checked": checked, "ms": ms}


def Event_pair():
    import ancora_cutile_b200 as anc
    return anc.Event(), anc.Event()


# ------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3", choices=["qwen3", "moe"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-grad-leg", action="store_true", help="skip the N > 1 gradient reduce-scatter check")
    ap.add_argument("--dump-digests", default=None, help="write per-tensor fingerprints of the bf16 parameters and of the owned float32 masters to this file (rank r > 0: FILE.rankR)")
    ap.add_argument("--layers", type=int, default=None, help="profiling only: fewer layers")
    ap.add_argument("--vocab", type=int, default=None, help="profiling only: smaller vocabulary")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    shp, wl_name = workload_shapes(args.workload, args.layers, args.vocab)
    muon_names = route(shp)
    total_params = int(sum(int(np.prod(s)) for s in shp.values()))
    config = {"workload": wl_name, "params": total_params, "muon_matrices": len(muon_names),
              "grad_dtype": "bf16", "ns": "polar-express x5", "adamw_rounding": "philox-sr",
              "parallelism": f"zero1x{world}" if world > 1 else "single",
              "l2": "state (7 GB) is far larger than L2; no flush needed"}

    # exchange of the updated bf16 parameters: "nccl_overlap" (default) or "nccl" (after the step)
    xmode = os.environ.get("ANCORA_EXCHANGE", "nccl_overlap")
    config["exchange"] = ("none" if world == 1 else ("NCCL all-gather per unit on a second stream"
                                                     if xmode == "nccl_overlap" else "NCCL all-gather after the step"))

    if args.impl == "reference":
        if rank != 0:
            return
        # a whole step when the caller asks for one or two, else a quarter of the layers per step so
        # that warm-up + steps end within minutes
        n_layers = 1 + max(int(n.split(".")[1]) for n in muon_names)
        layers = n_layers if args.steps <= 2 else max(1, n_layers // 4)
        cb = cpu_arm(shp, muon_names, total_params, max(args.steps, 1), min(args.warmup, 1), layers)
        print(json.dumps({
            "impl": "reference", "metric": "hybrid_optimizer_step_params_per_s", "value": cb["value"],
            "unit": "params/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import ancora_cutile_b200 as anc
    from ancora_cutile_b200 import shapes as S
    from ancora_cutile_b200.zero1 import Comm, nccl_unique_id

    anc.set_device(local_rank)
    ctx = anc.get_context()
    comm = None
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
        # NCCL may print its version banner on stdout; keep stdout for the one JSON line
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            box = [nccl_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            comm = Comm(ctx, box[0], rank, world)
            comm.barrier(ctx.stream)
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    if world > 1 and os.environ.get("ANCORA_RESERVE_SMS"):
        ctx.reserve_sms(int(os.environ["ANCORA_RESERVE_SMS"]))
        config["reserved_sms"] = int(os.environ["ANCORA_RESERVE_SMS"])
    anc.set_polar_express(True)
    params = S.synthetic_params(shp, seed=0)
    no_decay = tuple(n for n, s in shp.items() if len(s) == 1)
    eng = anc.ResidentHybrid(params, muon_names, no_decay_names=no_decay, adamw_kw=ADAMW_KW, muon_kw=MUON_KW,
                             grad_dtype="bf16", rounding="sr", seed=SEED_SR, rank=rank, world=world,
                             comm=comm, schedule=anc.PE_SCHEDULE, ctx=ctx)
    del params
    eng.nccl_overlap = world > 1 and xmode == "nccl_overlap"
    # synthetic bf16 gradients, written into the page-locked staging views and uploaded once
    pin = eng.pinned_grads()
    S.synthetic_grads_bf16(shp, seed=1, out=pin)
    eng.upload_grads(pin, ctx.stream)
    # synthetic optimizer state: m ~ N(0,1e-4), v = |N(0,1e-6)|, momentum ~ N(0,1e-3).
    # Each tensor's state comes from its own seeded stream and only the range this rank owns is
    # uploaded, so the state (and therefore the result) does not depend on the number of ranks.
    names = list(shp)
    for idx, name in enumerate(names):
        lo, hi = eng.owned_range(name)
        if hi <= lo:
            continue
        n = int(np.prod(shp[name]))
        r = np.random.default_rng(1000 + idx)
        if name in eng.a_off:
            o = eng.a_off[name] + lo - eng.a_begin
            eng.a_m.slice_elems(o, hi - lo).upload((r.standard_normal(n, dtype=np.float32) * np.float32(1e-4))[lo:hi])
            eng.a_v.slice_elems(o, hi - lo).upload(np.abs(r.standard_normal(n, dtype=np.float32) * np.float32(1e-6))[lo:hi])
        else:
            eng.m_buf.slice_elems(eng.m_own_off[name], n).upload(r.standard_normal(n, dtype=np.float32) * np.float32(1e-3))
    ctx.sync()

    if eng.muon is not None:
        eng.muon.set_timing(True)
    e0, e1 = anc.Event(), anc.Event()

    for _ in range(args.warmup):
        eng.step(ctx.stream)
    barrier()
    if eng.muon is not None:
        eng.muon.last_timing()          # drop the warm-up spans
    sampler = ClockSampler(local_rank)
    sampler.start()
    ns_ms = mom_ms = upd_ms = nrm_ms = adamw_ms = 0.0
    ns_flops = ns_flops_exec = 0.0
    gemm_launches = 0
    eng.trace_adamw = []                # CUDA events around each AdamW launch (no synchronisation)
    barrier()
    e0.record(ctx.stream)
    t_issue = time.perf_counter()
    for k in range(args.steps):
        eng.step(ctx.stream)            # with N > 1 this includes the exchange of the bf16 parameters
    e1.record(ctx.stream)
    host_issue_ms = (time.perf_counter() - t_issue) * 1e3 / args.steps   # time to ENQUEUE one step
    barrier()
    adamw_ms = sum(a0.elapsed_ms(a1) for a0, a1 in eng.trace_adamw)
    eng.trace_adamw = None
    if eng.muon is not None:
        t = eng.muon.last_timing()      # per-phase spans accumulated over the K timed steps
        ns_ms, mom_ms, upd_ms, nrm_ms = t["ns_ms"], t["momentum_ms"], t["update_ms"], t["normalize_ms"]
        ns_flops, ns_flops_exec, gemm_launches = t["ns_flops"], t["ns_flops_executed"], t["ns_launches"]
    clocks = sampler.stop()
    total_ms = max_over_ranks(e0.elapsed_ms(e1))
    ms_per_step = total_ms / args.steps
    value = total_params / (ms_per_step * 1e-3)
    K = args.steps
    peaks = measured_peaks()
    ns_tflops = ns_flops / (ns_ms * 1e-3) / 1e12 if ns_ms > 0 else 0.0
    ns_tflops_exec = ns_flops_exec / (ns_ms * 1e-3) / 1e12 if ns_ms > 0 else 0.0
    a_owned = min(eng.a_total, eng.a_end) - min(eng.a_total, eng.a_begin)
    adamw_gbs = 28.0 * a_owned / (adamw_ms / K * 1e-3) / 1e9 if adamw_ms > 0 else 0.0
    m_owned = eng.m_owned_elems
    elem_gbs = 24.0 * m_owned / ((mom_ms + upd_ms) / K * 1e-3) / 1e9 if (mom_ms + upd_ms) > 0 else 0.0
    n_groups = len([g for g in eng.groups if g["names"][rank]])
    # DRAM traffic of the GEMM launches: algorithmic bytes per matrix and iteration are 6MN + 8M^2
    # (operands once, outputs once); the measured ratio of DRAM bytes to that comes from an ncu capture.
    gemm_kernel = "ns_chain_kernel" if os.environ.get("ANCORA_NS_CHAIN", "1") != "0" else "ns_gemm_pair_kernel"
    gemm_alg_bytes = sum(len(g["names"][rank]) * MUON_KW["ns_steps"] *
                         (6 * g["shape"][0] * g["shape"][1] + 8 * g["shape"][0] ** 2) for g in eng.groups)
    launches_per_step = max(gemm_launches // K, 1)
    out = {
        "metric": "hybrid_optimizer_step_params_per_s", "value": value, "unit": "params/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config,
        # achieved = ALGORITHMIC (dense) FLOPs / time; the symmetric phases skip the tiles above the
        # diagonal, so the tensor cores execute fewer: that rate is reported beside it.  The timed
        # region is well under a second, so the peak is the burst cuBLAS figure.
        "roofline": {"bound": "tensor", "kernel": gemm_kernel, "achieved": ns_tflops,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": ns_tflops / peaks["bf16_tflops"],
                     "peak_kind": f"{peaks['src']} burst cuBLAS bf16 (sustained {peaks['bf16_tflops_sustained']})",
                     "frac_of_sustained": ns_tflops / peaks["bf16_tflops_sustained"],
                     "executed_flops_per_step": ns_flops_exec / K, "achieved_executed": ns_tflops_exec,
                     "frac_executed": ns_tflops_exec / peaks["bf16_tflops"],
                     "traffic": GEMM_TRAFFIC_RATIO * gemm_alg_bytes / launches_per_step,
                     "traffic_note": "bytes per launch: ncu dram read+write = %.2f x algorithmic bytes "
                                     "(capture named in traffic_source), scaled by matrices processed" % GEMM_TRAFFIC_RATIO,
                     "traffic_source": GEMM_TRAFFIC_SOURCE,
                     "algorithmic_bytes_per_launch": gemm_alg_bytes / launches_per_step,
                     "flops_per_step": ns_flops / K, "ms_per_step": ns_ms / K, "launches_per_step": gemm_launches // K},
        "adamw": {"bound": "hbm", "achieved": adamw_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                  "frac": adamw_gbs / peaks["hbm_gbs"], "frac_of_8tbs_nominal": adamw_gbs / 8000.0,
                  "bytes_per_param": 28, "params": a_owned, "ms_per_step": adamw_ms / K},
        "muon_elementwise": {"bound": "hbm", "achieved": elem_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": elem_gbs / peaks["hbm_gbs"], "bytes_per_param": 24,
                             "momentum_ms": mom_ms / K, "update_ms": upd_ms / K, "normalize_ms": nrm_ms / K},
        "clocks": clocks,
        "host_issue_ms_per_step": host_issue_ms,
        # per step: 3 GEMM launches per iteration and group, momentum + finalize + update per group, AdamW
        "gpu_launches": (gemm_launches // K) + 3 * n_groups + 1,
        # arena groups of the Muon parameters = all-gathers per step besides AdamW's (from four ranks on the
        # largest shape group is two arena groups, exchanged one after the other)
        "muon_arena_groups": len(eng.groups),
        "state_bytes_per_gpu": eng.state_bytes() + (eng.muon.scratch_bytes() if eng.muon else 0),
    }

    # ---- gradient producer (accumulate + SR downcast in one sweep) on an arena of the AdamW slice's
    # size, timed alone after the step loop: float32 accumulator, bf16 contribution, bf16 output ----
    if a_owned > 0:
        from ancora_cutile_b200 import kernels as K_
        g_acc = anc.DBuf.zeros((a_owned,), np.float32, ctx)
        g_src = anc.DBuf.zeros((a_owned,), np.uint16, ctx)
        g_out = anc.DBuf.zeros((a_owned,), np.uint16, ctx)
        reps = 10
        for i in range(3 + reps):
            if i == 3:
                e0.record(ctx.stream)
            K_.grad_accumulate(g_acc, g_src, g_out, a_owned, src_dtype="bf16", rounding="sr", seed=SEED_SR + 1,
                               step=i, elem_offset=eng.a_begin, stream=ctx.stream, ctx=ctx)
        e1.record(ctx.stream)
        ctx.sync()
        gp_ms = e0.elapsed_ms(e1) / reps
        gp_gbs = 12.0 * a_owned / (gp_ms * 1e-3) / 1e9
        out["grad_producer"] = {"bound": "hbm", "kernel": "grad_accumulate_kernel", "achieved": gp_gbs,
                                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gp_gbs / peaks["hbm_gbs"],
                                "bytes_per_elem": 12, "elems": a_owned, "ms": gp_ms,
                                "note": "timed alone, arena larger than L2, not part of ms_per_step"}
        for b in (g_acc, g_src, g_out):
            b.free()

    # ---- end-to-end: host gradients in, bf16 weights out, through the public call path ----
    if not args.no_e2e:
        h2d = d2h = 0
        for _ in range(2):
            eng.step_host(pin, ctx.stream)
        barrier()
        t0 = time.perf_counter()
        e0.record(ctx.stream)
        traces = []
        for _ in range(args.steps):
            tr = {}
            _, h2d, d2h = eng.step_host(pin, ctx.stream, trace=tr)     # synchronises: the result is on the host
            traces.append(tr)
        e1.record(ctx.stream)
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        e2e_ms = max_over_ranks(max(e0.elapsed_ms(e1) / args.steps, wall_ms))
        # where one step's time goes on this rank (device clock, ms from the start of the call, mean over
        # the timed steps): the copies run on their own streams beside the compute stream
        keys = [k for k in traces[0] if traces[0][k] is not None and k != "gathers"]
        brk = {k: float(np.mean([t[k] for t in traces])) for k in keys}
        if traces[-1].get("gathers"):
            brk["gathers_last_step"] = traces[-1]["gathers"]      # [group, start ms, end ms] of each all-gather
        brk["pcie_gbs_each_way"] = h2d / (max(brk["h2d_done_ms"], brk["d2h_done_ms"]) * 1e-3) / 1e9
        out["e2e"] = {"value": total_params / (e2e_ms * 1e-3), "unit": "params/s", "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "breakdown": brk,
                      "api": "HybridOptimizer.step_and_fetch -> ResidentHybrid.step_host: page-locked bf16 "
                             "gradients in, updated bf16 parameters out, pipelined per unit on 3 streams "
                             "(+ the NCCL all-gathers on a 4th when N > 1)"}
    # ---- gradient reduce-scatter feeding the ZeRO-1 owners (N > 1): every rank holds its own local
    # gradients for all parameters; float32 accumulate -> NCCL reduce-scatter -> bf16 downcast, checked on
    # every element this rank owns against the float64 sum over ranks, twice for repeatability ----
    if world > 1 and not args.no_grad_leg:
        out_rs = grad_reduce_scatter_leg(eng, pin, rank, world, ctx)
        box = [None] * world
        dist.all_gather_object(box, out_rs)
        out["grad_reduce_scatter"] = {
            "max_rel_err": max(b["max_rel_err"] for b in box), "tolerance": 2.0 ** -8,
            "repeatable_bits": all(b["repeatable_bits"] for b in box),
            "elements_checked": sum(b["elements_checked"] for b in box), "ms": max(b["ms"] for b in box),
            "what": "finalize_grads(reduce=True): bf16 grads -> f32 accumulators -> ncclReduceScatter(f32) -> "
                    "bf16 RNE of sum/world; compared with the float64 sum of the ranks' gradients"}
        eng.upload_grads(pin, ctx.stream)     # the step's own gradients again
    # Fingerprint of every updated bf16 parameter, name by name (independent of the arena layout):
    # all ranks must agree, and runs with the same --steps/--warmup at different N print the same
    # value, which is the "bitwise identical to the 1-GPU result" check at full size.
    import hashlib
    bits, _ = eng.download_weights_bits(ctx.stream)
    hsh = hashlib.blake2b(digest_size=16)
    for name in shp:
        hsh.update(np.ascontiguousarray(bits[name]).tobytes())
    digest = hsh.hexdigest()
    if args.dump_digests:
        # every rank writes its own view: the bf16 parameters it holds after the exchange and the
        # float32 masters of what it owns (which no exchange ever touches), so a mismatch can be
        # placed either in the owner's arithmetic or in the transport
        per = {name: hashlib.blake2b(np.ascontiguousarray(bits[name]).tobytes(), digest_size=8).hexdigest()
               for name in shp}
        masters = {name: [int(lo), int(hi), hashlib.blake2b(np.ascontiguousarray(v).tobytes(), digest_size=8).hexdigest()]
                   for name, (lo, hi, v) in eng.master().items()}
        path = args.dump_digests if rank == 0 else f"{args.dump_digests}.rank{rank}"
        with open(path, "w") as f:
            json.dump({"world": world, "rank": rank, "owner": {n: eng.m_owner.get(n, -1) for n in shp},
                       "digests": per, "masters": masters}, f)
    if dist is not None:
        box = [None] * world
        dist.all_gather_object(box, digest)
        out["params_agree_across_ranks"] = all(d == box[0] for d in box)
    out["params_blake2b"] = digest
    status = ctx.status()
    out["device_status"] = status

    if rank == 0 and world == 1 and not args.no_cpu:
        n_layers = 1 + max(int(n.split(".")[1]) for n in muon_names)
        out["cpu_baseline"] = cpu_arm(shp, muon_names, total_params, 1, 0, max(1, n_layers // 4))
    if rank == 0:
        print(json.dumps(out))
    eng.free()
    if comm is not None:
        comm.destroy()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

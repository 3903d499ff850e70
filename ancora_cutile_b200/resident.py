"""Device-resident hybrid optimizer state laid out in arenas, optionally ZeRO-1 sharded.

This is the engine under ``HybridOptimizer``; it is also what a resident model would hold
directly (the roles of ``opt[n]`` dicts + ResidentMuon/BatchedProjMuon in
ancora/model/resident_train.py:92-109,335-357 and resident_moe_model.py:116-141,357-374).

Layout in HBM (all device buffers are single allocations; tensors are views):
  AdamW  p16 : one bf16 arena, every tensor at its 64-aligned global offset, padded to
               world * per_rank so the exchange is one in-place all-gather.
         p32, m, v : float32 arenas holding only this rank's slice [begin, end).
         g   : gradient arena, full size (each rank fills at least its slice).
  Muon   p16 : bf16 arena laid out [shape group][owner rank][matrix]; inside a group every
               rank's region has the same (padded) size, so a group is gathered in place.
         p32, buf : float32 arenas of the owned matrices only, [shape group][matrix].
         g   : gradient arena with the p16 layout (each rank fills at least its own).

The step is a sequence of UNITS -- the AdamW slice, then each Muon shape group (largest
first) -- so that a unit's exchange (and, in ``step_host``, its host copies) overlaps the
next unit's compute.
"""
import ctypes as C
import os

import numpy as np

from . import _lib as L
from .adamw import ResidentAdamW
from .bf16 import bits_to_f32, f32_to_bf16_bits
from .buffers import DBuf, Event, PinnedArray, get_context
from .muon import MuonPlan, _UNSET, _schedule
from .layout import ArenaLayout


def _numel(shape):
    return int(np.prod(shape, dtype=np.int64))


class ResidentHybrid:
    def __init__(self, params, muon_names, no_decay_names=(), adamw_kw=None, muon_kw=None,
                 grad_dtype="bf16", rounding="sr", seed=0, rank=0, world=1, comm=None,
                 schedule=_UNSET, max_batch=0, ctx=None):
        """params: {name: fp32 ndarray} (every rank passes the same dict).
        comm: zero1.Comm; the updated bf16 parameters are exchanged with one NCCL all-gather per
        unit, issued on a second stream as soon as the unit is computed (``nccl_overlap``; set it
        to False for plain all-gathers after the step)."""
        self.ctx = ctx or get_context()
        self.rank, self.world, self.comm = int(rank), int(world), comm
        self.grad_dtype, self.rounding, self.seed = grad_dtype, rounding, int(seed)
        self.adamw_kw = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.01)
        self.adamw_kw.update(adamw_kw or {})
        self.muon_kw = dict(lr=0.02, momentum=0.95, nesterov=True, ns_steps=5)
        self.muon_kw.update(muon_kw or {})
        self._sched = schedule
        self.t = 0
        self.nccl_overlap = comm is not None
        gdt = np.uint16 if grad_dtype == "bf16" else np.float32
        self._gdt = np.dtype(gdt)
        lay = ArenaLayout({n: p.shape for n, p in params.items()}, muon_names, rank, world)
        self.layout = lay
        self.muon_names, self.adamw_names, self.shapes = lay.muon_names, lay.adamw_names, lay.shapes
        nd = set(no_decay_names)
        c = self.ctx
        W, R = self.world, self.rank

        # ---------------- AdamW arena
        self.a_off, self.a_total = lay.a_off, lay.a_total
        self.a_per, self.a_padded, self.a_begin, self.a_end = lay.a_per, lay.a_padded, lay.a_begin, lay.a_end
        self.a_p16 = DBuf.zeros((self.a_padded,), np.uint16, c)
        self.a_g = DBuf.zeros((self.a_padded,), gdt, c)
        self.a_p32 = DBuf.zeros((self.a_per,), np.float32, c)
        self.a_m = DBuf.zeros((self.a_per,), np.float32, c)
        self.a_v = DBuf.zeros((self.a_per,), np.float32, c)
        tensors = []
        for n in self.adamw_names:
            o, numel = self.a_off[n], _numel(self.shapes[n])
            flat = np.ascontiguousarray(params[n], dtype=np.float32).reshape(-1)
            self.a_p16.slice_elems(o, numel).upload(f32_to_bf16_bits(flat))
            lo, hi = max(o, self.a_begin), min(o + numel, self.a_end)
            if lo < hi:
                self.a_p32.slice_elems(lo - self.a_begin, hi - lo).upload(flat[lo - o:hi - o])
            # state pointers are relative to the slice: element i of the tensor lives at
            # arena[(o + i) - begin]; only indices inside [begin, end) are ever touched
            rel = (o - self.a_begin) * 4
            tensors.append(dict(g=self.a_g.ptr + o * self._gdt.itemsize, p32=self.a_p32.ptr + rel,
                                m=self.a_m.ptr + rel, v=self.a_v.ptr + rel, p16=self.a_p16.ptr + o * 2,
                                numel=numel, elem_offset=o,
                                wd=0.0 if n in nd else self.adamw_kw["wd"]))
        self._adamw_tensors = tensors
        self.adamw = ResidentAdamW(tensors, grad_dtype=grad_dtype, rounding=rounding, seed=seed, ctx=c)
        if W > 1:
            self.adamw.set_range(self.a_begin, self.a_end)

        # ---------------- Muon arenas: [group][owner][matrix]
        self.owner, self.load, self.m_owner = lay.owner, lay.load, lay.m_owner
        self.groups, self.m_off, self.m_own_off = lay.groups, lay.m_off, lay.m_own_off
        self.m_total, own = lay.m_total, lay.m_owned_elems
        self.m_p16 = DBuf.zeros((self.m_total,), np.uint16, c)
        self.m_g = DBuf.zeros((self.m_total,), gdt, c)
        self.m_p32 = DBuf.zeros((max(own, 64),), np.float32, c)
        self.m_buf = DBuf.zeros((max(own, 64),), np.float32, c)
        self.m_owned_elems = own
        ws = []
        for n in self.muon_names:
            w32 = np.ascontiguousarray(params[n], dtype=np.float32).reshape(-1)
            self.m_p16.slice_elems(self.m_off[n], w32.size).upload(f32_to_bf16_bits(w32))
            if self.m_owner[n] == R:
                self.m_p32.slice_elems(self.m_own_off[n], w32.size).upload(w32)
        for g in self.groups:                  # plan order = group order = arena order
            for n in g["names"][R]:
                K, N = self.shapes[n]
                ws.append(dict(buf=self.m_buf.ptr + self.m_own_off[n] * 4,
                               G=self.m_g.ptr + self.m_off[n] * self._gdt.itemsize,
                               p32=self.m_p32.ptr + self.m_own_off[n] * 4,
                               p16=self.m_p16.ptr + self.m_off[n] * 2, K=K, N=N))
        self.muon = MuonPlan(ws, grad_dtype=grad_dtype, max_batch=max_batch, ctx=c) if ws else None
        # Units of work, each a contiguous span of this rank's share of an arena:
        #   ("adamw", plan, begin, end)            arena-0 elements [begin, end)
        #   ("muon", plan group, first, count, arena group key, first inside the arena group)
        #                                          matrices [first, first+count) of a shape group of the plan
        self._gmap = lay.gmap
        self._pgroup = {}                      # shape key -> (plan group index, scratch batch)
        if self.muon is not None:
            for gi in range(self.muon.num_groups()):
                _, cap, M, Nn = self.muon.group_info(gi)
                self._pgroup[(M, Nn)] = (gi, cap)
        # step_host cuts units to at most this many elements: its run time is the transfer time of
        # all bytes plus the (transfer + compute) time of the LARGEST unit, so smaller units shorten
        # the pipeline's tail until the Newton-Schulz batches get too small to keep up with the uploads
        # (measured on the benchmark step: 64 MiB units 27.5 ms, 32 MiB 26.8 ms, 16 MiB 38.8 ms)
        self.host_chunk_elems = int(os.environ.get("ANCORA_HOST_CHUNK_ELEMS", 16 << 20))
        self._sub_plans = []
        self.units = self._make_units(None)
        self._host_units = None
        self._pin_g = None
        self._pin_w = None
        self._streams = None
        self._comm_stream = None

    # ---------------------------------------------------------------- locations
    def _loc(self, name):
        if name in self.a_off:
            return self.a_p16, self.a_g, self.a_off[name]
        return self.m_p16, self.m_g, self.m_off[name]

    def p16_view(self, name):
        """bf16 weight of ``name`` as a device view (what a forward pass would read)."""
        p16, _, o = self._loc(name)
        return p16.slice_elems(o, _numel(self.shapes[name]), self.shapes[name])

    def grad_view(self, name):
        _, g, o = self._loc(name)
        return g.slice_elems(o, _numel(self.shapes[name]), self.shapes[name])

    def owned_range(self, name):
        """(start, stop) flat element range of ``name`` whose state this rank holds."""
        n = _numel(self.shapes[name])
        if name in self.a_off:
            o = self.a_off[name]
            lo, hi = max(o, self.a_begin), min(o + n, self.a_end)
            return (lo - o, hi - o) if lo < hi else (0, 0)
        return (0, n) if self.m_owner[name] == self.rank else (0, 0)

    def _make_units(self, max_elems):
        """AdamW first, then shape groups by descending size (the last unit's exchange or
        copy-out is the one nothing overlaps, so the smallest goes last).  ``max_elems`` cuts
        units into sub-ranges of at most that many elements (host pipelining)."""
        units = []
        caps = {key: cap for key, (_, cap) in self._pgroup.items()}
        for u in self.layout.make_units(caps, max_elems):
            if u[0] == "muon":
                g = self._gmap[u[1]]
                units.append(("muon", self._pgroup[g["shape"]][0], g["plan_first"] + u[2], u[3], u[1], u[2]))
            elif max_elems is None:
                units.append(("adamw", self.adamw, u[1], u[2]))
            else:                              # a sub-range of the slice gets a plan of its own
                pl = ResidentAdamW(self._adamw_tensors, grad_dtype=self.grad_dtype, rounding=self.rounding,
                                   seed=self.seed, ctx=self.ctx)
                pl.set_range(u[1], u[2])
                self._sub_plans.append(pl)
                units.append(("adamw", pl, u[1], u[2]))
        return units

    def unit_span(self, unit):
        """(arena index, element offset, element count) of the unit's span in the bf16
        parameter / gradient arenas (arena 0 = AdamW, 1 = Muon)."""
        if unit[0] == "adamw":
            return 0, unit[2], unit[3] - unit[2]
        g = self._gmap[unit[4]]
        return 1, g["base"] + self.rank * g["per"] + unit[5] * g["elems"], unit[3] * g["elems"]

    # ---------------------------------------------------------------- the step
    def _compute_unit(self, unit, si):
        a, m = self.adamw_kw, self.muon_kw
        if unit[0] == "adamw":
            tr = getattr(self, "trace_adamw", None)
            if tr is not None:                 # benchmark hook: CUDA events around the launch
                e0, e1 = Event(), Event()
                e0.record(si)
            unit[1].step(si, a["lr"], a["betas"][0], a["betas"][1], a["eps"], t=self.t)
            if tr is not None:
                e1.record(si)
                tr.append((e0, e1))
        else:
            self.muon.step_range(unit[1], unit[2], unit[3], si, m["lr"], m["momentum"], m["nesterov"],
                                 m["ns_steps"], _schedule(self._sched))

    def _events(self, n):
        if not hasattr(self, "_evpool"):
            self._evpool = []
        while len(self._evpool) < n:
            self._evpool.append(Event())
        return self._evpool[:n]

    def step(self, si=None, exchange=True):
        """One optimizer step on stream ``si``; asynchronous.  With world > 1 the updated bf16
        parameters are exchanged by NCCL all-gathers, one per arena group."""
        si = si or self.ctx.stream
        self.t += 1
        multi = exchange and self.world > 1
        if multi and self.nccl_overlap:
            # NCCL all-gather of each unit on a second stream as soon as the unit is computed
            cs = self._comm_stream_handle()
            if getattr(self, "_overlap_for", None) is not self.units:
                self._overlap_steps = self.layout.exchange_schedule(
                    ["adamw" if u[0] == "adamw" else u[4] for u in self.units])
                self._overlap_for = self.units
            steps = self._overlap_steps
            evs = self._events(sum(1 for op in steps if op[0] == "gather") + 1)
            lib = L.lib()
            k = 0
            for op, what in steps:
                if op == "compute":
                    self._compute_unit(self.units[what], si)
                    continue
                ev = evs[k]
                k += 1
                ev.record(si)
                L.check(lib.anc_stream_wait_event(cs, ev.handle))
                self._gather_group(what, cs)
            done = evs[k]
            done.record(cs)
            L.check(lib.anc_stream_wait_event(si, done.handle))
            return
        for u in self.units:
            self._compute_unit(u, si)
        if multi:
            self.exchange(si)

    def step_part(self, kind, si=None, exchange=True):
        """Only the AdamW units (kind "adamw": advances the step number ``t``) or only the Muon
        units (kind "muon"), for callers that drive the two sub-optimizers separately as the
        reference's ``opt.muon.step`` / ``opt.adamw.step`` do (ancora/optim/hybrid.py:45-47)."""
        assert kind in ("adamw", "muon")
        si = si or self.ctx.stream
        if kind == "adamw":
            self.t += 1
        for u in self.units:
            if u[0] == kind:
                self._compute_unit(u, si)
        if exchange and self.world > 1:
            assert self.comm is not None, "world > 1 needs a communicator"
            if kind == "adamw":
                self.comm.allgather_bf16(self.a_p16.ptr, self.a_per, si)
            else:
                for g in self.groups:
                    self.comm.allgather_bf16(self.m_p16.ptr + g["base"] * 2, g["per"], si)

    def upload_full_grads(self, grads, si=None):
        """Host -> device copy of ALL gradients (a data-parallel replica's local gradients, to
        be summed across ranks by ``reduce_scatter_grads``)."""
        self._stage_grads(grads)
        pa, pm, _ = self._pin_g
        it = self._gdt.itemsize
        L.check(L.lib().anc_h2d(self.ctx.handle, self.a_g.ptr, pa.ptr, self.a_padded * it, si or None, 0))
        L.check(L.lib().anc_h2d(self.ctx.handle, self.m_g.ptr, pm.ptr, self.m_total * it, si or None, 0))

    def reduce_scatter_grads(self, si=None):
        """Data-parallel gradient reduction feeding the ZeRO-1 owners: every rank holds local
        gradients for all parameters in its gradient arenas; afterwards each rank's own AdamW
        slice and own Muon matrices hold the sum over ranks (NCCL reduce-scatter per unit, in
        place, in the gradient dtype).  Nothing in the reference corresponds to it (single
        GPU); it is the producer side of the sharded step."""
        assert self.comm is not None, "reduce_scatter_grads needs an NCCL communicator"
        it = self._gdt.itemsize
        self.comm.reduce_scatter_grads(self.a_g.ptr, self.a_per, self.grad_dtype, si)
        for g in self.groups:
            self.comm.reduce_scatter_grads(self.m_g.ptr + g["base"] * it, g["per"], self.grad_dtype, si)

    # ---------------------------------------------------------------- gradient accumulation
    def enable_grad_accumulation(self):
        """Allocates float32 accumulators with the layout of the two gradient arenas (4 B/param).
        Micro-batch gradients keep arriving in the gradient arenas as before (``upload_grads``,
        ``grad_view``); ``accumulate_grads`` folds them into the accumulators and
        ``finalize_grads`` turns the sum into the bf16 gradients the step reads."""
        assert self.grad_dtype == "bf16", "with float32 gradients accumulate in the gradient arenas themselves"
        if getattr(self, "acc_a", None) is None:
            self.acc_a = DBuf.zeros((self.a_padded,), np.float32, self.ctx)
            self.acc_m = DBuf.zeros((self.m_total,), np.float32, self.ctx)
            self.acc_count = 0

    def accumulate_grads(self, si=None):
        """acc += the gradients now in the gradient arenas (one sweep per arena, all regions: a
        data-parallel replica holds local gradients for every parameter)."""
        from . import kernels
        for acc, g, n in ((self.acc_a, self.a_g, self.a_padded), (self.acc_m, self.m_g, self.m_total)):
            kernels.grad_accumulate(acc, g, None, n, src_dtype="bf16", stream=si, ctx=self.ctx)
        self.acc_count += 1

    def finalize_grads(self, si=None, scale=None, rounding="sr", seed=None, reduce=True):
        """Last micro-batch: acc += the gradients in the arenas, then (world > 1 and ``reduce``) the
        float32 accumulators are reduce-scattered to their ZeRO-1 owners, and one sweep per arena
        writes bf16(acc * scale) back into the gradient arenas and clears the accumulators.
        ``scale`` defaults to 1 / (micro-batches * world).  Stochastic rounding draws from the
        producer's own Philox stream (seed + 1 of the step's by default, counter = position in the
        arena and the number of the step about to run), so it is reproducible for a fixed world size."""
        from . import kernels
        self.accumulate_grads(si)
        multi = reduce and self.world > 1
        if multi:
            assert self.comm is not None, "finalize_grads needs an NCCL communicator to reduce"
            self.comm.reduce_scatter_grads(self.acc_a.ptr, self.a_per, "f32", si)
            for g in self.groups:
                self.comm.reduce_scatter_grads(self.acc_m.ptr + g["base"] * 4, g["per"], "f32", si)
        if scale is None:
            scale = 1.0 / (self.acc_count * (self.world if multi else 1))
        seed = (self.seed + 1) if seed is None else seed
        # the Muon arena's stream starts after the AdamW arena's, so no two elements share a counter
        for acc, g, n, off in ((self.acc_a, self.a_g, self.a_padded, 0),
                               (self.acc_m, self.m_g, self.m_total, self.a_padded)):
            kernels.grad_accumulate(acc, None, g, n, elem_offset=off, scale=scale, rounding=rounding, seed=seed,
                                    step=self.t + 1, zero_after=True, stream=si, ctx=self.ctx)
        self.acc_count = 0

    # ---------------------------------------------------------------- graph replay
    def capture_step(self, si=None, horizon=4096):
        """Captures one whole step into a CUDA graph whose replay advances the optimizer by one
        step: AdamW's step number and scalars come from device memory (a schedule for the next
        ``horizon`` steps is uploaded here), everything else in the step has fixed arguments.
        Call after at least one eager ``step`` (first calls allocate); hyper-parameters are
        and the stochastic-rounding seed are frozen into the graph.  The device step counter is
        mirrored on the host (``_graph_next``): eager steps or ``load_state_dict`` between replays
        move ``t`` away from it, and ``replay_step`` then points the device counter at ``t + 1``
        again before launching (or asks for a new capture when that step lies outside the
        uploaded schedule or the seed changed)."""
        si = si or self.ctx.stream
        a = self.adamw_kw
        self.ctx.sync(si)
        self.adamw.set_schedule(self.t + 1, horizon, a["lr"], a["betas"][0], a["betas"][1], a["eps"])
        self._graph_first = self.t + 1
        self._graph_limit = self.t + horizon
        self._graph_next = self.t + 1
        self._graph_seed = self.seed
        lib = L.lib()
        L.check(lib.anc_graph_begin(self.ctx.handle, si))
        try:
            for u in self.units:
                if u[0] == "adamw":
                    u[1].step_scheduled(si, advance=True)
                else:
                    self._compute_unit(u, si)
            if self.world > 1:
                self.exchange(si)
        finally:
            g = C.c_void_p()
            L.check(lib.anc_graph_end(self.ctx.handle, si, C.byref(g)))
        if getattr(self, "_graph", None):
            lib.anc_graph_destroy(self._graph)
        self._graph = g

    def replay_step(self, si=None):
        """One optimizer step by replaying the captured graph (asynchronous)."""
        assert getattr(self, "_graph", None), "capture_step first"
        si = si or self.ctx.stream
        if self.seed != self._graph_seed:
            raise RuntimeError("the stochastic-rounding seed changed since capture_step: capture again")
        if not (self._graph_first <= self.t + 1 <= self._graph_limit):
            raise RuntimeError(f"step {self.t + 1} lies outside the captured schedule "
                               f"[{self._graph_first}, {self._graph_limit}]: capture_step again")
        if self._graph_next != self.t + 1:
            # an eager step or a restored state moved the step number since the last replay
            self.adamw.set_counter(self.t + 1, si)
            self._graph_next = self.t + 1
        self.t += 1
        self._graph_next += 1
        L.check(L.lib().anc_graph_launch(self.ctx.handle, self._graph, si))

    def exchange(self, si=None):
        """NCCL path: one in-place all-gather per unit."""
        assert self.comm is not None, "world > 1 needs a communicator"
        self.comm.allgather_bf16(self.a_p16.ptr, self.a_per, si)
        for g in self.groups:
            self.comm.allgather_bf16(self.m_p16.ptr + g["base"] * 2, g["per"], si)

    # ---------------------------------------------------------------- host traffic
    def pinned_grads(self):
        """Page-locked host staging for the gradients, one numpy view per name, laid out like
        the device gradient arenas so that one copy per unit moves everything."""
        if self._pin_g is None:
            pa = PinnedArray((self.a_padded,), self._gdt, self.ctx.device)
            pm = PinnedArray((self.m_total,), self._gdt, self.ctx.device)
            views = {}
            for n in self.adamw_names + self.muon_names:
                src = pa if n in self.a_off else pm
                o = self.a_off[n] if n in self.a_off else self.m_off[n]
                views[n] = src.array[o:o + _numel(self.shapes[n])].reshape(self.shapes[n])
            self._pin_g = (pa, pm, views)
        return self._pin_g[2]

    def _stage_grads(self, grads, names=None):
        views = self.pinned_grads()
        if grads is views:
            return                            # the caller filled the staging views themselves
        for n in (views if names is None else names):
            v = views[n]
            g = grads[n]
            if isinstance(g, np.ndarray) and g.ctypes.data == v.ctypes.data and g.dtype == v.dtype:
                continue                      # caller wrote straight into the staging view
            if self._gdt == np.uint16 and np.asarray(g).dtype != np.uint16:
                g = f32_to_bf16_bits(np.asarray(g, np.float32))
            np.copyto(v, np.asarray(g, dtype=self._gdt).reshape(v.shape))

    def _h2d_unit(self, unit, stream):
        pa, pm, _ = self._pin_g
        arena, off, n = self.unit_span(unit)
        it = self._gdt.itemsize
        dev, host = (self.a_g, pa) if arena == 0 else (self.m_g, pm)
        if n:
            L.check(L.lib().anc_h2d(self.ctx.handle, dev.ptr + off * it, host.ptr + off * it, n * it,
                                    stream or None, 0))
        return n * it

    def _d2h_unit(self, unit, stream):
        wa, wm = self._pin_w
        arena, off, n = self.unit_span(unit)
        dev, host = (self.a_p16, wa) if arena == 0 else (self.m_p16, wm)
        if n:
            L.check(L.lib().anc_d2h(self.ctx.handle, host.ptr + off * 2, dev.ptr + off * 2, n * 2,
                                    stream or None, 0))
        return n * 2

    def upload_grads(self, grads, si=None, kind=None):
        """Host -> device copy of this rank's share of the gradients (asynchronous); ``kind``
        ("adamw" or "muon") restricts it to one sub-optimizer's tensors."""
        names = None if kind is None else (self.adamw_names if kind == "adamw" else self.muon_names)
        self._stage_grads(grads, names)
        return sum(self._h2d_unit(u, si) for u in self.units if kind is None or u[0] == kind)

    def _ensure_host_side(self):
        if self._pin_w is None:
            self._pin_w = (PinnedArray((self.a_padded,), np.uint16, self.ctx.device),
                           PinnedArray((self.m_total,), np.uint16, self.ctx.device))
        if self._streams is None:
            ss = []
            for _ in range(2):
                s = C.c_void_p()
                L.check(L.lib().anc_stream_create(self.ctx.handle, C.byref(s)))
                ss.append(s.value)
            self._streams = ss
        self.pinned_grads()
        if self._host_units is None:
            self._host_units = self._make_units(self.host_chunk_elems)

    def _weight_views(self):
        """{name: uint16 view of the page-locked weight arenas}; the arenas never move, so the views are
        made once (a few hundred numpy slices per call would sit between two pipelined steps)."""
        cached = getattr(self, "_wviews", None)
        if cached is not None and cached[0] is self._pin_w:
            return dict(cached[1])
        wa, wm = self._pin_w
        out = {}
        for n in self.adamw_names + self.muon_names:
            src = wa if n in self.a_off else wm
            o = self.a_off[n] if n in self.a_off else self.m_off[n]
            out[n] = src.array[o:o + _numel(self.shapes[n])].reshape(self.shapes[n])
        self._wviews = (self._pin_w, out)
        return dict(out)

    def _comm_stream_handle(self):
        if self._comm_stream is None:
            st = C.c_void_p()
            L.check(L.lib().anc_stream_create(self.ctx.handle, C.byref(st)))
            self._comm_stream = st.value
        return self._comm_stream

    def _gather_group(self, what, stream):
        """In-place all-gather of one arena group ("adamw" or a Muon shape key) on ``stream``."""
        if what == "adamw":
            self.comm.allgather_bf16(self.a_p16.ptr, self.a_per, stream)
        else:
            g = self._gmap[what]
            self.comm.allgather_bf16(self.m_p16.ptr + g["base"] * 2, g["per"], stream)

    def step_host(self, grads, si=None, trace=None):
        """The whole round trip a host-API caller makes, pipelined unit by unit on three
        streams: gradients host -> device, the step, this rank's updated bf16 parameters device ->
        host; with world > 1 each arena group's all-gather is issued on a fourth stream as soon as
        the group's last unit is computed.  Returns ({name: uint16 view of page-locked memory},
        bytes copied in, bytes copied out) after synchronising.  With world > 1 only the
        parameters this rank owns are copied out.

        trace: a dict that receives, in milliseconds from the start of the call on the device
        clock, when the last upload, the last compute, the last download and the last all-gather
        finished, plus the host time spent staging and enqueueing."""
        import time
        si = si or self.ctx.stream
        t_host0 = time.perf_counter()
        self._ensure_host_side()
        self._stage_grads(grads)
        t_staged = time.perf_counter()
        s_in, s_out = self._streams
        self.t += 1
        units = self._host_units
        nu = len(units)
        multi = self.world > 1
        if multi:
            assert self.comm is not None, "world > 1 needs a communicator"
            if getattr(self, "_host_sched_for", None) is not units:
                self._host_sched = self.layout.exchange_schedule(
                    ["adamw" if u[0] == "adamw" else u[4] for u in units])
                self._host_sched_for = units
            sched = self._host_sched
            cs = self._comm_stream_handle()
        else:
            sched = [("compute", k) for k in range(nu)]
            cs = None
        ng = sum(1 for op in sched if op[0] == "gather")
        evs = self._events(3 * nu + ng + 8)
        ev_in, ev_c, ev_out = evs[:nu], evs[nu:2 * nu], evs[2 * nu:3 * nu]
        ev_g = evs[3 * nu:3 * nu + ng]
        start, m_in, m_c, m_out, m_x, end, done_x = evs[3 * nu + ng:3 * nu + ng + 7]
        start.record(si)                       # copies may not overtake work queued earlier on si
        lib = L.lib()
        L.check(lib.anc_stream_wait_event(s_in, start.handle))
        L.check(lib.anc_stream_wait_event(s_out, start.handle))
        if cs is not None:
            L.check(lib.anc_stream_wait_event(cs, start.handle))
        h2d = d2h = 0
        gi = 0
        gspans = []
        for op, what in sched:
            if op == "gather":
                ev = ev_g[gi]
                gi += 1
                ev.record(si)
                L.check(lib.anc_stream_wait_event(cs, ev.handle))
                if trace is not None:              # when each all-gather ran, on the device clock
                    g0, g1 = Event(), Event()
                    g0.record(cs)
                self._gather_group(what, cs)
                if trace is not None:
                    g1.record(cs)
                    gspans.append((str(what), g0, g1))
                continue
            k, u = what, units[what]
            h2d += self._h2d_unit(u, s_in)
            ev_in[k].record(s_in)
            L.check(lib.anc_stream_wait_event(si, ev_in[k].handle))
            self._compute_unit(u, si)
            ev_c[k].record(si)
            L.check(lib.anc_stream_wait_event(s_out, ev_c[k].handle))
            d2h += self._d2h_unit(u, s_out)
            ev_out[k].record(s_out)
        if trace is not None:
            m_in.record(s_in)
            m_c.record(si)
            m_out.record(s_out)
            if cs is not None:
                m_x.record(cs)
        if cs is not None:
            done_x.record(cs)
            L.check(lib.anc_stream_wait_event(si, done_x.handle))
        L.check(lib.anc_stream_wait_event(si, ev_out[nu - 1].handle))   # s_out is in order: the last covers all
        if trace is not None:
            end.record(si)
        t_enq = time.perf_counter()
        self.ctx.sync(si)
        if trace is not None:
            trace.update(h2d_done_ms=start.elapsed_ms(m_in), compute_done_ms=start.elapsed_ms(m_c),
                         d2h_done_ms=start.elapsed_ms(m_out),
                         exchange_done_ms=start.elapsed_ms(m_x) if cs is not None else None,
                         total_ms=start.elapsed_ms(end), units=nu,
                         gathers=[[w, start.elapsed_ms(a), start.elapsed_ms(b)] for w, a, b in gspans],
                         host_stage_ms=(t_staged - t_host0) * 1e3, host_enqueue_ms=(t_enq - t_staged) * 1e3)
        for _, a, b in gspans:
            a.destroy()
            b.destroy()
        return self._weight_views(), h2d, d2h

    def download_weights_bits(self, si=None, sync=True):
        """Device -> host copy of every bf16 parameter into page-locked memory; returns
        ({name: uint16 view}, bytes copied)."""
        self._ensure_host_side()
        wa, wm = self._pin_w
        d2h = L.lib().anc_d2h
        L.check(d2h(self.ctx.handle, wa.ptr, self.a_p16.ptr, self.a_padded * 2, si or None, 0))
        L.check(d2h(self.ctx.handle, wm.ptr, self.m_p16.ptr, self.m_total * 2, si or None, 0))
        if sync:
            self.ctx.sync(si)
        return self._weight_views(), (self.a_padded + self.m_total) * 2

    def weights(self):
        bits, _ = self.download_weights_bits()
        return {n: bits_to_f32(b) for n, b in bits.items()}

    def master(self):
        """fp32 masters this rank holds: {name: (start, stop, flat values)}; with world == 1
        that is every tensor in full."""
        out = {}
        a32 = self.a_p32.to_numpy()
        for n in self.adamw_names:
            s, e = self.owned_range(n)
            if e > s:
                o = self.a_off[n] + s - self.a_begin
                out[n] = (s, e, a32[o:o + e - s].copy())
        if self.muon is not None:
            m32 = self.m_p32.to_numpy()
            for n in self.muon_names:
                if self.m_owner[n] == self.rank:
                    k = _numel(self.shapes[n])
                    out[n] = (0, k, m32[self.m_own_off[n]:self.m_own_off[n] + k].copy())
        return out

    # ---------------------------------------------------------------- save / resume
    def state_dict(self):
        """Everything needed to resume this rank bit-exactly: the fp32 arenas it owns, both
        bf16 parameter arenas, the step counter and the SR seed, plus the layout facts a loader
        checks.  (The reference has no optimizer-state save/load; its state is only readable
        through master()/weights(), adamw.py:100-105.)"""
        self.ctx.sync()
        return {
            "format": 1, "rank": self.rank, "world": self.world, "t": self.t, "seed": self.seed,
            "grad_dtype": self.grad_dtype, "rounding": self.rounding,
            "a_total": self.a_total, "a_begin": self.a_begin, "a_end": self.a_end, "m_total": self.m_total,
            "names": list(self.adamw_names) + list(self.muon_names),
            "a_p32": self.a_p32.to_numpy(), "a_m": self.a_m.to_numpy(), "a_v": self.a_v.to_numpy(),
            "m_p32": self.m_p32.to_numpy(), "m_buf": self.m_buf.to_numpy(),
            "a_p16": self.a_p16.to_numpy(), "m_p16": self.m_p16.to_numpy(),
        }

    def load_state_dict(self, sd):
        """Restores a ``state_dict`` made by an engine built from the same parameter names and
        shapes with the same world size and rank."""
        want = dict(format=1, rank=self.rank, world=self.world, a_total=self.a_total, a_begin=self.a_begin,
                    a_end=self.a_end, m_total=self.m_total, grad_dtype=self.grad_dtype, rounding=self.rounding,
                    names=list(self.adamw_names) + list(self.muon_names))
        for k, v in want.items():
            if sd.get(k) != v:
                raise ValueError(f"state_dict does not fit this engine: {k} is {sd.get(k)!r}, expected {v!r}")
        for name in ("a_p32", "a_m", "a_v", "m_p32", "m_buf", "a_p16", "m_p16"):
            buf, arr = getattr(self, name), np.ascontiguousarray(sd[name])
            if arr.shape != tuple(buf.shape) or arr.dtype != buf.dtype:
                raise ValueError(f"state_dict[{name}] has shape {arr.shape} {arr.dtype}")
            buf.upload(arr)
        self.t = int(sd["t"])
        self.seed = int(sd["seed"])
        self.adamw.seed = self.seed
        for pl in self._sub_plans:
            pl.seed = self.seed

    def state_bytes(self):
        return sum(b.nbytes for b in (self.a_p16, self.a_g, self.a_p32, self.a_m, self.a_v,
                                      self.m_p16, self.m_g, self.m_p32, self.m_buf))

    def free(self):
        self.ctx.sync()
        if getattr(self, "_graph", None):
            L.lib().anc_graph_destroy(self._graph)
            self._graph = None
        self.adamw.free()
        for pl in self._sub_plans:
            pl.free()
        self._sub_plans = []
        if self.muon is not None:
            self.muon.free()
            self.muon = None
        for b in (self.a_p16, self.a_g, self.a_p32, self.a_m, self.a_v, self.m_p16, self.m_g,
                  self.m_p32, self.m_buf, getattr(self, "acc_a", None), getattr(self, "acc_m", None)):
            if b is not None:
                b.free()
        self.acc_a = self.acc_m = None
        for grp in (self._pin_g[:2] if self._pin_g else ()), (self._pin_w or ()):
            for p in grp:
                p.free()
        self._pin_g = self._pin_w = None
        if self._streams:
            for s in self._streams:
                L.lib().anc_stream_destroy(self.ctx.handle, s)
            self._streams = None
        if self._comm_stream:
            L.lib().anc_stream_destroy(self.ctx.handle, self._comm_stream)
            self._comm_stream = None
        for e in getattr(self, "_evpool", []):
            e.destroy()
        self._evpool = []

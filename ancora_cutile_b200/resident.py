"""Device-resident hybrid optimizer state laid out in arenas, optionally ZeRO-1 sharded.

This is the engine under ``HybridOptimizer``; it is also what a resident model would hold
directly (the roles of ``opt[n]`` dicts + ResidentMuon/BatchedProjMuon in
ancora/model/resident_train.py:92-109,335-357 and resident_moe_model.py:116-141,357-374).

Layout in HBM (all device buffers are single allocations; tensors are views):
  AdamW  p16 : one bf16 arena, every tensor at its 64-aligned global offset, padded to
               world * per_rank so the exchange is one in-place all-gather.
         p32, m, v : float32 arenas holding only this rank's slice [begin, end).
         g   : gradient arena, full size (each rank fills at least its slice).
  Muon   p16 : bf16 arena ordered by owner rank, each rank's region padded to the largest.
         p32, buf : float32 arenas of the owned matrices only.
         g   : gradient arena over all matrices (each rank fills at least its own).
"""
import numpy as np

from . import _lib as L
from .adamw import ResidentAdamW, align_up
from .bf16 import bits_to_f32, f32_to_bf16_bits
from .buffers import DBuf, PinnedArray, get_context
from .muon import MuonPlan, _UNSET, _schedule
from .zero1 import greedy_partition, ns_cost, slice_bounds


class ResidentHybrid:
    def __init__(self, params, muon_names, no_decay_names=(), adamw_kw=None, muon_kw=None,
                 grad_dtype="bf16", rounding="sr", seed=0, rank=0, world=1, comm=None,
                 schedule=_UNSET, max_batch=0, ctx=None):
        """params: {name: fp32 ndarray} (every rank passes the same dict)."""
        self.ctx = ctx or get_context()
        self.rank, self.world, self.comm = int(rank), int(world), comm
        self.grad_dtype, self.rounding, self.seed = grad_dtype, rounding, int(seed)
        self.adamw_kw = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.01)
        self.adamw_kw.update(adamw_kw or {})
        self.muon_kw = dict(lr=0.02, momentum=0.95, nesterov=True, ns_steps=5)
        self.muon_kw.update(muon_kw or {})
        self._sched = schedule
        self.t = 0
        gdt = np.uint16 if grad_dtype == "bf16" else np.float32
        self._gdt = np.dtype(gdt)
        mset = set(muon_names)
        self.muon_names = [n for n in params if n in mset]
        self.adamw_names = [n for n in params if n not in mset]
        self.shapes = {n: tuple(p.shape) for n, p in params.items()}
        nd = set(no_decay_names)
        c = self.ctx

        # ---------------- AdamW arena
        self.a_off, off = {}, 0
        for n in self.adamw_names:
            self.a_off[n] = off
            off = align_up(off + int(np.prod(self.shapes[n], dtype=np.int64)), 64)
        self.a_total = off
        self.a_per, self.a_padded = slice_bounds(max(off, 64), self.world, 64)
        self.a_begin, self.a_end = self.rank * self.a_per, (self.rank + 1) * self.a_per
        self.a_p16 = DBuf.zeros((self.a_padded,), np.uint16, c)
        self.a_g = DBuf.zeros((self.a_padded,), gdt, c)
        self.a_p32 = DBuf.zeros((self.a_per,), np.float32, c)
        self.a_m = DBuf.zeros((self.a_per,), np.float32, c)
        self.a_v = DBuf.zeros((self.a_per,), np.float32, c)
        tensors = []
        for n in self.adamw_names:
            o, numel = self.a_off[n], int(np.prod(self.shapes[n], dtype=np.int64))
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
        self.adamw = ResidentAdamW(tensors, grad_dtype=grad_dtype, rounding=rounding, seed=seed, ctx=c)
        if self.world > 1:
            self.adamw.set_range(self.a_begin, self.a_end)

        # ---------------- Muon arenas
        costs = [ns_cost(*self.shapes[n]) for n in self.muon_names]
        self.owner, self.load = greedy_partition(costs, self.world)
        sizes = {n: int(np.prod(self.shapes[n], dtype=np.int64)) for n in self.muon_names}
        region = [0] * self.world
        self.m_off = {}                      # offset inside the owner's region
        for n, r in zip(self.muon_names, self.owner):
            self.m_off[n] = region[r]
            region[r] += sizes[n]
        self.m_per = align_up(max(region + [64]), 64)
        self.m_p16 = DBuf.zeros((self.m_per * self.world,), np.uint16, c)
        self.m_g = DBuf.zeros((self.m_per * self.world,), gdt, c)
        mine = max(region[self.rank], 64)
        self.m_p32 = DBuf.zeros((mine,), np.float32, c)
        self.m_buf = DBuf.zeros((mine,), np.float32, c)
        ws = []
        self.m_owner = dict(zip(self.muon_names, self.owner))
        for n in self.muon_names:
            r, K, N = self.m_owner[n], *self.shapes[n]
            g_off = r * self.m_per + self.m_off[n]
            w32 = np.ascontiguousarray(params[n], dtype=np.float32).reshape(-1)
            self.m_p16.slice_elems(g_off, sizes[n]).upload(f32_to_bf16_bits(w32))
            if r == self.rank:
                self.m_p32.slice_elems(self.m_off[n], sizes[n]).upload(w32)
                ws.append(dict(buf=self.m_buf.ptr + self.m_off[n] * 4, G=self.m_g.ptr + g_off * self._gdt.itemsize,
                               p32=self.m_p32.ptr + self.m_off[n] * 4, p16=self.m_p16.ptr + g_off * 2,
                               K=K, N=N))
        self.muon = MuonPlan(ws, grad_dtype=grad_dtype, max_batch=max_batch, ctx=c) if ws else None
        self._pin_g = None
        self._pin_w = None

    # ---------------------------------------------------------------- locations
    def p16_view(self, name):
        """bf16 weight of ``name`` as a device view (what a forward pass would read)."""
        n = int(np.prod(self.shapes[name], dtype=np.int64))
        if name in self.a_off:
            return self.a_p16.slice_elems(self.a_off[name], n, self.shapes[name])
        return self.m_p16.slice_elems(self.m_owner[name] * self.m_per + self.m_off[name], n, self.shapes[name])

    def grad_view(self, name):
        n = int(np.prod(self.shapes[name], dtype=np.int64))
        if name in self.a_off:
            return self.a_g.slice_elems(self.a_off[name], n, self.shapes[name])
        return self.m_g.slice_elems(self.m_owner[name] * self.m_per + self.m_off[name], n, self.shapes[name])

    def owned_range(self, name):
        """(start, stop) flat element range of ``name`` whose state this rank holds."""
        n = int(np.prod(self.shapes[name], dtype=np.int64))
        if name in self.a_off:
            o = self.a_off[name]
            lo, hi = max(o, self.a_begin), min(o + n, self.a_end)
            return (lo - o, hi - o) if lo < hi else (0, 0)
        return (0, n) if self.m_owner[name] == self.rank else (0, 0)

    # ---------------------------------------------------------------- the step
    def step(self, si=None, exchange=True):
        """One optimizer step on stream ``si``; asynchronous.  With world > 1 the updated
        bf16 parameters are all-gathered at the end (``exchange``)."""
        self.t += 1
        a, m = self.adamw_kw, self.muon_kw
        if self.muon is not None:
            self.muon.step(si, m["lr"], m["momentum"], m["nesterov"], m["ns_steps"], _schedule(self._sched))
        self.adamw.step(si, a["lr"], a["betas"][0], a["betas"][1], a["eps"], t=self.t)
        if exchange and self.world > 1:
            self.exchange(si)

    def exchange(self, si=None):
        assert self.comm is not None, "world > 1 needs a communicator"
        self.comm.allgather_bf16(self.a_p16.ptr, self.a_per, si)
        self.comm.allgather_bf16(self.m_p16.ptr, self.m_per, si)

    # ---------------------------------------------------------------- host traffic
    def pinned_grads(self):
        """Page-locked host staging for the gradients, one numpy view per name, laid out like
        the device gradient arenas so that one copy per arena moves everything."""
        if self._pin_g is None:
            pa = PinnedArray((self.a_padded,), self._gdt)
            pm = PinnedArray((self.m_per * self.world,), self._gdt)
            views = {}
            for n in self.adamw_names:
                k = int(np.prod(self.shapes[n], dtype=np.int64))
                views[n] = pa.array[self.a_off[n]:self.a_off[n] + k].reshape(self.shapes[n])
            for n in self.muon_names:
                k = int(np.prod(self.shapes[n], dtype=np.int64))
                o = self.m_owner[n] * self.m_per + self.m_off[n]
                views[n] = pm.array[o:o + k].reshape(self.shapes[n])
            self._pin_g = (pa, pm, views)
        return self._pin_g[2]

    def upload_grads(self, grads, si=None):
        """Host -> device copy of this rank's share of the gradients (asynchronous)."""
        views = self.pinned_grads()
        pa, pm, _ = self._pin_g
        for n, v in views.items():
            g = grads[n]
            if isinstance(g, np.ndarray) and g.ctypes.data == v.ctypes.data and g.dtype == v.dtype:
                continue                      # caller wrote straight into the staging view
            if self._gdt == np.uint16 and np.asarray(g).dtype != np.uint16:
                g = f32_to_bf16_bits(np.asarray(g, np.float32))
            np.copyto(v, np.asarray(g, dtype=self._gdt).reshape(v.shape))
        it = self._gdt.itemsize
        h2d = L.lib().anc_h2d
        # AdamW: the owned slice; Muon: the owned region
        L.check(h2d(self.ctx.handle, self.a_g.ptr + self.a_begin * it, pa.ptr + self.a_begin * it,
                    self.a_per * it, si or None, 0))
        L.check(h2d(self.ctx.handle, self.m_g.ptr + self.rank * self.m_per * it,
                    pm.ptr + self.rank * self.m_per * it, self.m_per * it, si or None, 0))
        return 2 * 0 + (self.a_per + self.m_per) * it

    def download_weights_bits(self, si=None, sync=True):
        """Device -> host copy of every bf16 parameter into page-locked memory; returns
        ({name: uint16 view}, bytes copied)."""
        if self._pin_w is None:
            self._pin_w = (PinnedArray((self.a_padded,), np.uint16),
                           PinnedArray((self.m_per * self.world,), np.uint16))
        wa, wm = self._pin_w
        d2h = L.lib().anc_d2h
        L.check(d2h(self.ctx.handle, wa.ptr, self.a_p16.ptr, self.a_padded * 2, si or None, 0))
        L.check(d2h(self.ctx.handle, wm.ptr, self.m_p16.ptr, self.m_per * self.world * 2, si or None, 0))
        if sync:
            self.ctx.sync(si)
        out = {}
        for n in self.adamw_names:
            k = int(np.prod(self.shapes[n], dtype=np.int64))
            out[n] = wa.array[self.a_off[n]:self.a_off[n] + k].reshape(self.shapes[n])
        for n in self.muon_names:
            k = int(np.prod(self.shapes[n], dtype=np.int64))
            o = self.m_owner[n] * self.m_per + self.m_off[n]
            out[n] = wm.array[o:o + k].reshape(self.shapes[n])
        return out, (self.a_padded + self.m_per * self.world) * 2

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
                    k = int(np.prod(self.shapes[n], dtype=np.int64))
                    out[n] = (0, k, m32[self.m_off[n]:self.m_off[n] + k].copy())
        return out

    def state_bytes(self):
        return sum(b.nbytes for b in (self.a_p16, self.a_g, self.a_p32, self.a_m, self.a_v,
                                      self.m_p16, self.m_g, self.m_p32, self.m_buf))

    def free(self):
        self.adamw.free()
        if self.muon is not None:
            self.muon.free()
            self.muon = None
        for b in (self.a_p16, self.a_g, self.a_p32, self.a_m, self.a_v, self.m_p16, self.m_g,
                  self.m_p32, self.m_buf):
            b.free()
        for grp in (self._pin_g[:2] if self._pin_g else ()), (self._pin_w or ()):
            for p in grp:
                p.free()
        self._pin_g = self._pin_w = None

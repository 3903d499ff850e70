"""Muon with the reference's Python API (ancora/optim/muon.py), backed by the library's
batched Muon plan: momentum+Nesterov -> packed bf16 -> Frobenius normalise -> tcgen05
Newton-Schulz chain -> master update + bf16 refresh, all on the device.

Classes and their reference counterparts:
  Muon             host-API optimizer, params/grads as numpy dicts      muon.py:287-318
  ResidentMuon     one resident weight over caller-owned p32/p16        muon.py:164-204
  BatchedProjMuon  all resident 2-D weights, batched by NS shape        muon.py:207-284
  MuonScratch      kept for signature parity; the plan owns its scratch muon.py:137-161
  DeviceMuon       one device-resident weight that owns all its buffers muon.py:88-135
  ExpertMuonScratch  caller-visible scratch of the batched expert chain ancora/kernels/moe.py:404-421

Coefficients: callers that pass no ``schedule`` get the process-wide default selected by
``set_polar_express`` (Keller unless switched on), as in the reference.
"""
import ctypes as C

import numpy as np

from . import _lib as L
from . import muon_ns
from .bf16 import bits_to_f32, f32_to_bf16_bits
from .buffers import DBuf, dev_ptr, get_context

_GRAD = {"bf16": L.GRAD_BF16, "f32": L.GRAD_F32}
_UNSET = object()


def _check_aligned(K, N):
    assert K % muon_ns.NTM == 0 and N % muon_ns.NTM == 0, f"Muon weight ({K},{N}) tile-misaligned"


class MuonPlan:
    """ctypes handle of one anc_muon_plan over a fixed list of weights."""

    def __init__(self, weights, grad_dtype="f32", my_rank=0, max_batch=0, ctx=None):
        self.ctx = ctx or get_context()
        arr = (L.MuonWeight * max(len(weights), 1))()
        outs = (L.MuonOutputs * max(len(weights), 1))()
        for i, w in enumerate(weights):
            _check_aligned(w["K"], w["N"])
            arr[i] = L.MuonWeight(dev_ptr(w["buf"]), dev_ptr(w["G"]), dev_ptr(w["p32"]), dev_ptr(w["p16"]),
                                  int(w["K"]), int(w["N"]), int(w.get("owner", -1)), 0)
            # optional fused post-step outputs: MXFP8 re-quant (fp8 + fp8_scale), transposed bf16 copy,
            # MXFP8 in the transposed (N,K) layout (fp8_t + fp8_scale_t)
            outs[i] = L.MuonOutputs(dev_ptr(w.get("fp8")), dev_ptr(w.get("fp8_scale")), dev_ptr(w.get("p16_t")),
                                    dev_ptr(w.get("fp8_t")), dev_ptr(w.get("fp8_scale_t")))
        h = C.c_void_p()
        L.check(L.lib().anc_muon_plan_create_ex(self.ctx.handle, arr, outs, len(weights), _GRAD[grad_dtype],
                                                int(my_rank), int(max_batch or 0), C.byref(h)))
        self.handle = h

    def step(self, si, lr, momentum, nesterov, ns_steps, schedule, eps=1e-7):
        co = muon_ns.coeff_list(schedule, ns_steps)
        flat = (C.c_float * max(3 * ns_steps, 1))(*[float(x) for t in co for x in t])
        L.check(L.lib().anc_muon_step(self.handle, float(lr), float(momentum), int(bool(nesterov)),
                                      int(ns_steps), flat, float(eps), C.c_void_p(si or None)))

    def num_groups(self):
        n = C.c_int()
        L.check(L.lib().anc_muon_plan_num_groups(self.handle, C.byref(n)))
        return n.value

    def group_info(self, g):
        """(weights in the group, largest range the scratch holds, M, N)."""
        info = (C.c_int32 * 4)()
        L.check(L.lib().anc_muon_plan_group_info(self.handle, int(g), info))
        return tuple(info)

    def step_range(self, g, first, count, si, lr, momentum, nesterov, ns_steps, schedule, eps=1e-7):
        co = muon_ns.coeff_list(schedule, ns_steps)
        flat = (C.c_float * max(3 * ns_steps, 1))(*[float(x) for t in co for x in t])
        L.check(L.lib().anc_muon_step_range(self.handle, int(g), int(first), int(count), float(lr),
                                            float(momentum), int(bool(nesterov)), int(ns_steps), flat,
                                            float(eps), C.c_void_p(si or None)))

    def set_timing(self, on):
        L.check(L.lib().anc_muon_plan_set_timing(self.handle, int(bool(on))))

    def last_timing(self):
        ms = (C.c_float * 4)()
        fl = (C.c_double * 2)()
        nl = C.c_int()
        L.check(L.lib().anc_muon_plan_last_timing(self.handle, ms, fl, C.byref(nl)))
        return dict(momentum_ms=ms[0], normalize_ms=ms[1], ns_ms=ms[2], update_ms=ms[3],
                    ns_flops=fl[0], ns_flops_executed=fl[1], ns_launches=nl.value)

    def scratch_bytes(self):
        b = C.c_uint64()
        L.check(L.lib().anc_muon_plan_scratch_bytes(self.handle, C.byref(b)))
        return b.value

    def free(self):
        if self.handle:
            L.lib().anc_muon_plan_destroy(self.handle)
            self.handle = None


def _schedule(explicit):
    return muon_ns._DEFAULT_SCHEDULE if explicit is _UNSET else explicit


class MuonScratch:
    """Signature-compatible stand-in: the batched plan allocates and shares its own packed
    scratch, so this only records the shapes it was asked to cover."""

    def __init__(self, shapes):
        self.shapes = [tuple(int(x) for x in s) for s in shapes]

    def nbytes(self):
        return 0

    def free(self):
        pass


class DeviceMuon:
    """Device-resident Muon over ONE 2-D weight that owns its buffers (ancora/optim/muon.py:88-135):
    fp32 master ``p32``, one momentum buffer ``buf``, the bf16 weight ``p16`` the forward reads.
    ``step(g_dev, si)`` takes the (K,N) float32 device gradient and runs momentum -> Newton-Schulz ->
    update -> bf16 refresh on the device, asynchronously.  The reference's per-weight scratch
    (``u, gA, gA2, gB, scr, gBX, recip``) lives inside the plan here."""

    def __init__(self, W, lr=0.02, momentum=0.95, ns_steps=5, grad_dtype="f32", schedule=_UNSET, ctx=None):
        W = np.asarray(W)
        assert W.ndim == 2, f"Muon is for 2D matrices, got {W.shape}"
        K, N = W.shape
        _check_aligned(K, N)
        self.ctx = ctx or get_context()
        self.K, self.N, self.tr = K, N, K > N
        self.M, self.Nn = (N, K) if self.tr else (K, N)
        self.lr = lr
        self.lr_scale = lr * max(1.0, K / N) ** 0.5
        self.mom, self.ns = momentum, ns_steps
        w32 = np.ascontiguousarray(W, dtype=np.float32)
        self.p32 = DBuf(w32, self.ctx)
        self.p16 = DBuf(f32_to_bf16_bits(w32), self.ctx)
        self._inner = ResidentMuon(self.p32, self.p16, K, N, None, momentum, ns_steps, grad_dtype=grad_dtype,
                                   schedule=schedule, ctx=self.ctx)
        self.buf = self._inner.buf

    def step(self, g_dev, si):
        self._inner.step(g_dev, si, lr=self.lr)

    def master(self):
        return self.p32.to_numpy()

    def weights(self):
        return bits_to_f32(self.p16.to_numpy())

    def free(self):
        self._inner.free()
        self.p32.free()
        self.p16.free()


class ExpertMuonScratch:
    """Scratch of the batched expert Newton-Schulz chain with the reference's attribute names
    (ancora/kernels/moe.py:404-421): ``u`` (E*M, N) holds the packed momentum input and receives
    the orthogonalised output, ``gA, gB`` (E*M, M), ``gBX`` (E*M, N), ``recip`` (E, 1); pass them
    to ``newton_schulz_resident_e(sc.u, sc.gA, sc.gA2, sc.gB, sc.gBX, sc.recip, E, M, N, si)`` as the
    reference's GroupedMoEFFN.step does (moe.py:583-586).  ``gA2`` is a one-row stand-in: the fused
    chain never materialises A@A.  N defaults to M (the reference's square experts); rectangular
    experts pass N explicitly."""

    def __init__(self, E, M, N=None, ctx=None):
        N = M if N is None else N
        assert M <= N and M % muon_ns.NTM == 0 and N % muon_ns.NTN == 0, f"expert shape ({M},{N}) tile-misaligned"
        self.ctx = ctx or get_context()
        self.E, self.M, self.N = E, M, N
        Z = lambda *s: DBuf.zeros(s, np.uint16, self.ctx)
        self.gA, self.gB = Z(E * M, M), Z(E * M, M)
        self.gA2 = Z(1, 8)
        self.gBX, self.u = Z(E * M, N), Z(E * M, N)
        self.recip = DBuf.zeros((E, 1), np.float32, self.ctx)

    def nbytes(self):
        return sum(b.nbytes for b in (self.gA, self.gA2, self.gB, self.gBX, self.u, self.recip))

    def free(self):
        for b in (self.gA, self.gA2, self.gB, self.gBX, self.u, self.recip):
            b.free()


class ResidentMuon:
    """Per-weight Muon over the caller's p32/p16 (the forward reads p16 in place).  The only
    persistent state is the momentum buffer ``buf`` (8 B/param with p32, muon.py:165-166)."""

    def __init__(self, p32, p16, K, N, scratch=None, momentum=0.95, ns_steps=5, grad_dtype="f32",
                 schedule=_UNSET, ctx=None):
        _check_aligned(K, N)
        self.ctx = ctx or get_context()
        self.p32, self.p16, self.K, self.N, self.sc = p32, p16, K, N, scratch
        self.tr = K > N
        self.M, self.Nn = (N, K) if self.tr else (K, N)
        self.shape_scale = max(1.0, K / N) ** 0.5
        self.mom, self.ns, self.grad_dtype, self._sched = momentum, ns_steps, grad_dtype, schedule
        self.buf = DBuf.zeros((K, N), np.float32, self.ctx)
        self._plan, self._gptr = None, None

    def step(self, g_dev, si, lr=0.02):
        gp = dev_ptr(g_dev)
        if self._plan is None or gp != self._gptr:
            if self._plan is not None:
                self._plan.free()
            self._plan = MuonPlan([dict(buf=self.buf, G=gp, p32=self.p32, p16=self.p16, K=self.K, N=self.N)],
                                  grad_dtype=self.grad_dtype, ctx=self.ctx)
            self._gptr = gp
        self._plan.step(si, lr, self.mom, True, self.ns, _schedule(self._sched))

    def free(self):
        if self._plan is not None:
            self._plan.free()
            self._plan = None
        self.buf.free()


class BatchedProjMuon:
    """Model-level batched Muon over all resident 2-D weights (muon.py:207-284).

    weights: list of {buf, p32, p16, G, K, N, lid}.  ``chunk`` caps how many matrices of one
    shape share a Newton-Schulz batch (None = the whole group; the reference's 8 was sized
    for a 16 GB laptop GPU).  ``scope=k`` steps each k-layer bucket through its own plan;
    results are bitwise identical to the global grouping because every matrix's tiles,
    K order and reductions are independent of batch composition."""

    def __init__(self, weights, momentum=0.95, ns_steps=5, chunk=None, scope=None, grad_dtype="f32",
                 schedule=_UNSET, ctx=None):
        self.ctx = ctx or get_context()
        self.mom, self.ns, self._sched = momentum, ns_steps, schedule
        buckets = {}
        for w in weights:
            _check_aligned(w["K"], w["N"])
            key = 0 if scope is None else w.get("lid", 0) // scope
            buckets.setdefault(key, []).append(w)
        self.plans = [MuonPlan(ws, grad_dtype=grad_dtype, max_batch=chunk or 0, ctx=self.ctx)
                      for _, ws in sorted(buckets.items())]

    def step(self, si, lr=0.02):
        for p in self.plans:
            p.step(si, lr, self.mom, True, self.ns, _schedule(self._sched))

    def free(self):
        for p in self.plans:
            p.free()
        self.plans = []


class Muon:
    """fp32-master Muon for 2-D matrix params.  params: {name: (R,C) fp32 ndarray}.
    Same constructor and methods as the reference's host class (muon.py:287-318); the state
    lives on the device and every step runs there.  ``device``/``si`` are accepted for
    signature parity (the reference's device=True round-trip path is the slow one it kept as
    a negative result, muon.py:45-52)."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, device=False, si=None,
                 grad_dtype="f32", schedule=_UNSET, max_batch=0, ctx=None):
        self.lr, self.mom, self.nesterov, self.ns = lr, momentum, nesterov, ns_steps
        self.device, self.si = device, si
        self.ctx = ctx or get_context()
        self.grad_dtype, self._sched = grad_dtype, schedule
        gdt = np.uint16 if grad_dtype == "bf16" else np.float32
        self.st = {}
        ws = []
        for n, p in params.items():
            assert p.ndim == 2, f"Muon is for 2D matrices, {n} is {p.shape}"
            K, N = p.shape
            _check_aligned(K, N)
            w32 = np.ascontiguousarray(p, dtype=np.float32)
            s = dict(shape=(K, N), K=K, N=N, p32=DBuf(w32, self.ctx), p16=DBuf(f32_to_bf16_bits(w32), self.ctx),
                     buf=DBuf.zeros((K, N), np.float32, self.ctx), G=DBuf.zeros((K, N), gdt, self.ctx))
            self.st[n] = s
            ws.append(s)
        self._plan = MuonPlan(ws, grad_dtype=grad_dtype, max_batch=max_batch, ctx=self.ctx) if ws else None

    def _grad_host(self, g):
        if self.grad_dtype == "f32":
            return np.ascontiguousarray(g, dtype=np.float32)
        g = np.asarray(g)
        return np.ascontiguousarray(g) if g.dtype == np.uint16 else f32_to_bf16_bits(g.astype(np.float32))

    def step(self, grads, stream_int=None):
        si = stream_int if stream_int is not None else self.si
        if self._plan is None:
            return
        for n, s in self.st.items():
            s["G"].upload(self._grad_host(grads[n]), si, sync=False)     # one sync at the end of the step
        self._plan.step(si, self.lr, self.mom, self.nesterov, self.ns, _schedule(self._sched))
        self.ctx.sync(si)
        self.ctx.check_status()

    def weights(self):
        return {n: bits_to_f32(s["p16"].to_numpy()) for n, s in self.st.items()}

    def master(self):
        return {n: s["p32"].to_numpy() for n, s in self.st.items()}

    def free(self):
        if self._plan is not None:
            self._plan.free()
            self._plan = None
        for s in self.st.values():
            for k in ("p32", "p16", "buf", "G"):
                s[k].free()
        self.st = {}

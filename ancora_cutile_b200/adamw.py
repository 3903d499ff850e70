"""AdamW with the reference's Python API (ancora/optim/adamw.py:69-109), backed by the
library's single-launch multi-tensor kernel.

Differences from the reference, all opt-in except the launch structure:
* one kernel launch covers every tensor (the reference launches once per tensor);
* ``grad_dtype="bf16"`` reads bf16 gradients (28 B/param); the default "f32" keeps the
  reference's float32 gradients so its own test formulas hold to their tolerance;
* ``rounding="sr"`` writes the bf16 parameter copy by Philox stochastic rounding keyed on
  (seed, step, global element index); the default "rne" is the reference's cast.

``ResidentAdamW`` is the device-resident form the models use (grads already on the
device, caller-owned p32/p16, no host traffic, asynchronous): the role of the
``ct.launch(si, ..., _adamw, ...)`` loops in ancora/model/resident_train.py:349-353 and
resident_model.py:160-166.
"""
import ctypes as C

import numpy as np

from . import _lib as L
from .bf16 import bits_to_f32, f32_to_bf16_bits
from .buffers import DBuf, dev_ptr, get_context

C64 = 64  # the reference flattens every tensor to (numel//64, 64) (adamw.py:20)
_GRAD = {"bf16": L.GRAD_BF16, "f32": L.GRAD_F32}
_ROUND = {"rne": L.ROUND_RNE, "sr": L.ROUND_SR}


def step_scalars(lr, b1, b2, eps, t):
    """float32 scalars of step t, materialised once: 1-beta is the float32 subtraction the
    reference kernel performs (adamw.py:34-35), the bias corrections are computed in
    double and cast (adamw.py:90-91,97)."""
    f = np.float32
    return L.AdamWScalars(float(f(b1)), float(f(1.0) - f(b1)), float(f(b2)), float(f(1.0) - f(b2)),
                          float(f(eps)), float(f(lr)),
                          float(f(1.0 / (1.0 - b1 ** t))), float(f(1.0 / (1.0 - b2 ** t))))


def align_up(x, a):
    return (x + a - 1) // a * a


class ResidentAdamW:
    """Multi-tensor AdamW over device buffers the caller owns.

    tensors: list of dicts {g, p32, p16, numel, wd[, m, v][, elem_offset]}; m/v are
    allocated (zeroed) here when absent and freed by ``free()``.  Offsets into the global
    arena default to a running sum with each tensor aligned to 64 elements.
    """

    def __init__(self, tensors, grad_dtype="bf16", rounding="rne", seed=0, ctx=None):
        self.ctx = ctx or get_context()
        self.grad_dtype, self.rounding, self.seed = grad_dtype, rounding, int(seed)
        self._owned = []
        arr = (L.AdamWTensor * max(len(tensors), 1))()
        off = 0
        self.offsets = []
        for i, t in enumerate(tensors):
            n = int(t["numel"])
            eo = int(t["elem_offset"]) if "elem_offset" in t else off
            off = align_up(eo + n, C64)
            self.offsets.append(eo)
            m, v = t.get("m"), t.get("v")
            if m is None:
                m = DBuf.zeros((n,), np.float32, self.ctx); self._owned.append(m)
            if v is None:
                v = DBuf.zeros((n,), np.float32, self.ctx); self._owned.append(v)
            arr[i] = L.AdamWTensor(dev_ptr(t["g"]), dev_ptr(t["p32"]), dev_ptr(m), dev_ptr(v),
                                   dev_ptr(t["p16"]), n, eo, float(t.get("wd", 0.0)), 0.0)
        self.arena_elems = off
        h = C.c_void_p()
        L.check(L.lib().anc_adamw_plan_create(self.ctx.handle, arr, len(tensors), _GRAD[grad_dtype],
                                              C.byref(h)))
        self.handle = h
        self.t = 0

    def set_range(self, begin, end):
        L.check(L.lib().anc_adamw_plan_set_range(self.handle, int(begin), int(end)))

    def step(self, si=None, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, t=None):
        """Asynchronous on ``si``.  ``t`` overrides the internal step counter."""
        if t is None:
            self.t += 1
            t = self.t
        s = step_scalars(lr, b1, b2, eps, t)
        L.check(L.lib().anc_adamw_step(self.handle, C.byref(s), _ROUND[self.rounding], self.seed, int(t),
                                       C.c_void_p(si or None)))

    def set_schedule(self, first_step, n, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8):
        """Uploads the scalars of steps first_step .. first_step+n-1 and sets the device step
        counter to first_step (for ``step_scheduled`` / graph replay)."""
        tab = (L.AdamWScalars * n)(*[step_scalars(lr, b1, b2, eps, first_step + k) for k in range(n)])
        L.check(L.lib().anc_adamw_plan_set_schedule(self.handle, tab, n, int(first_step)))

    def set_counter(self, step, si=None):
        """Points the device step counter at ``step`` (must lie inside the uploaded schedule)."""
        L.check(L.lib().anc_adamw_plan_set_counter(self.handle, int(step), C.c_void_p(si or None)))

    def step_scheduled(self, si=None, advance=True):
        """The step whose number is in the device counter; capturable in a CUDA graph."""
        L.check(L.lib().anc_adamw_step_scheduled(self.handle, _ROUND[self.rounding], self.seed,
                                                 int(bool(advance)), C.c_void_p(si or None)))

    def free(self):
        if self.handle:
            L.lib().anc_adamw_plan_destroy(self.handle)
            self.handle = None
        for b in self._owned:
            b.free()
        self._owned = []


class AdamW:
    """fp32-master AdamW.  params: {name: fp32 ndarray}.  no_decay: names with wd=0.
    step(grads, stream) uploads the gradients, runs one fused launch and synchronises
    (adamw.py:88-98); weights() returns the bf16-valued fp32 weights (adamw.py:100-102)."""

    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.01, no_decay=(),
                 grad_dtype="f32", rounding="rne", seed=0, ctx=None):
        self.lr, (self.b1, self.b2), self.eps, self.wd = lr, betas, eps, wd
        self.t = 0
        self.ctx = ctx or get_context()
        self.grad_dtype = grad_dtype
        gdt = np.uint16 if grad_dtype == "bf16" else np.float32
        self.st = {}
        tensors = []
        for name, p in params.items():
            flat = np.ascontiguousarray(p, dtype=np.float32).reshape(-1)
            n = flat.size
            s = dict(shape=p.shape, numel=n, wd=0.0 if name in no_decay else wd,
                     g=DBuf.zeros((n,), gdt, self.ctx),
                     m=DBuf.zeros((n,), np.float32, self.ctx), v=DBuf.zeros((n,), np.float32, self.ctx),
                     p32=DBuf(flat, self.ctx), p16=DBuf(f32_to_bf16_bits(flat), self.ctx))
            self.st[name] = s
            tensors.append(s)
        self._plan = ResidentAdamW(tensors, grad_dtype=grad_dtype, rounding=rounding, seed=seed, ctx=self.ctx)

    def _grad_host(self, g):
        if self.grad_dtype == "f32":
            return np.ascontiguousarray(g, dtype=np.float32).reshape(-1)
        g = np.asarray(g)
        if g.dtype == np.uint16:
            return np.ascontiguousarray(g).reshape(-1)
        return f32_to_bf16_bits(g.astype(np.float32)).reshape(-1)

    def step(self, grads, stream_int=None):
        self.t += 1
        # pageable host memory: the copy call returns once the source has been staged, so temporaries
        # are safe without a synchronisation per tensor (the reference syncs once, adamw.py:98)
        for name, s in self.st.items():
            s["g"].upload(self._grad_host(grads[name]), stream_int, sync=False)
        self._plan.step(stream_int, self.lr, self.b1, self.b2, self.eps, t=self.t)
        self.ctx.sync(stream_int)
        self.ctx.check_status()

    def weights(self):
        return {n: bits_to_f32(s["p16"].to_numpy()).reshape(s["shape"]) for n, s in self.st.items()}

    def master(self):
        return {n: s["p32"].to_numpy().reshape(s["shape"]) for n, s in self.st.items()}

    def moments(self):
        return {n: (s["m"].to_numpy().reshape(s["shape"]), s["v"].to_numpy().reshape(s["shape"]))
                for n, s in self.st.items()}

    def free(self):
        self._plan.free()
        for s in self.st.values():
            for k in ("g", "m", "v", "p32", "p16"):
                s[k].free()
        self.st = {}

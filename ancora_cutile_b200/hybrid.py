"""Muon + AdamW hybrid with the reference's API (ancora/optim/hybrid.py).

Routing is the reference's: Muon on 2-D hidden matrices, AdamW on everything else
(1-D gains, embedding, LM head).  State lives in device arenas (``ResidentHybrid``);
``step(grads, stream)`` stages the host gradients through page-locked memory, runs the
whole step on the device and synchronises, like the reference's host-API classes
(adamw.py:88-98).  ``muon_device`` and ``si`` are accepted for signature parity.

Extra keyword arguments (all default to the reference's behaviour):
  grad_dtype "f32" | "bf16"      gradient element type read by the kernels
  rounding   "rne" | "sr"        AdamW bf16 copy: round-to-nearest-even or Philox SR
  seed                           SR stream seed
  rank, world, comm              ZeRO-1 sharding over one node's GPUs
"""
import numpy as np

from .resident import ResidentHybrid


def default_is_muon(name, p):
    """2-D matrix that is not a norm gain / embedding / lm_head (hybrid.py:18-25)."""
    if p.ndim != 2:
        return False
    low = name.lower()
    if any(t in low for t in ("norm", "ln", "embed", "lm_head", "head", "wte", "wpe")):
        return False
    return True


class _Part:
    """View of one sub-optimizer (the reference exposes ``.muon`` and ``.adamw``)."""

    def __init__(self, owner, names, kw):
        self._o, self.names, self.kw = owner, names, kw

    @property
    def lr(self):
        return self.kw["lr"]

    @lr.setter
    def lr(self, v):
        self.kw["lr"] = v

    def weights(self):
        w = self._o.weights()
        return {n: w[n] for n in self.names}

    def master(self):
        m = self._o.master()
        return {n: m[n] for n in self.names if n in m}


class HybridOptimizer:
    def __init__(self, params, is_muon=default_is_muon, no_decay=None, muon_kw=None, adamw_kw=None,
                 si=None, muon_device=False, grad_dtype="f32", rounding="rne", seed=0,
                 rank=0, world=1, comm=None, schedule=None, max_batch=0, ctx=None):
        muon_kw = dict(lr=0.02, momentum=0.95, ns_steps=5, **(muon_kw or {}))
        adamw_kw = adamw_kw or dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.01)
        if no_decay is None:
            no_decay = lambda n, p: (p.ndim == 1)
        self.si = si
        self.muon_names = [n for n, p in params.items() if is_muon(n, p)]
        self.adamw_names = [n for n in params if n not in self.muon_names]
        for n in self.muon_names:
            assert params[n].ndim == 2, f"Muon is for 2D matrices, {n} is {params[n].shape}"
        from .muon import _UNSET
        self.engine = ResidentHybrid(
            params, self.muon_names,
            no_decay_names=tuple(n for n in self.adamw_names if no_decay(n, params[n])),
            adamw_kw=adamw_kw, muon_kw=muon_kw, grad_dtype=grad_dtype, rounding=rounding, seed=seed,
            rank=rank, world=world, comm=comm, schedule=_UNSET if schedule is None else schedule,
            max_batch=max_batch, ctx=ctx)
        self.muon = _Part(self, self.muon_names, self.engine.muon_kw)
        self.adamw = _Part(self, self.adamw_names, self.engine.adamw_kw)

    def step(self, grads, stream_int=None):
        si = stream_int if stream_int is not None else self.si
        e = self.engine
        e.upload_grads(grads, si)
        e.step(si)
        e.ctx.sync(si)
        e.ctx.check_status()

    def step_and_fetch(self, grads, stream_int=None):
        """step() and the read-back of the updated bf16 weights as ONE pipelined call: the
        gradient upload, the optimizer kernels and the download of finished parameters overlap
        unit by unit.  Returns {name: uint16 bf16 bit patterns} (views of page-locked memory,
        valid until the next call)."""
        si = stream_int if stream_int is not None else self.si
        bits, _, _ = self.engine.step_host(grads, si)
        self.engine.ctx.check_status()
        return bits

    def pinned_grads(self):
        """Page-locked numpy views, one per parameter, that ``step`` / ``step_and_fetch`` copy
        from without an extra host copy when the caller writes gradients straight into them."""
        return self.engine.pinned_grads()

    def weights(self):
        """bf16-valued fp32 weights for the next forward, per name."""
        return self.engine.weights()

    def master(self):
        """fp32 masters per name (with ZeRO-1: only what this rank owns, owned range only)."""
        out = {}
        for n, (s, e, flat) in self.engine.master().items():
            full = int(np.prod(self.engine.shapes[n], dtype=np.int64))
            out[n] = flat.reshape(self.engine.shapes[n]) if (s, e) == (0, full) else flat
        return out

    def state_dict(self):
        """Resumable optimizer state of this rank (see ResidentHybrid.state_dict)."""
        return self.engine.state_dict()

    def load_state_dict(self, sd):
        self.engine.load_state_dict(sd)

    def routing(self):
        return {"muon": list(self.muon_names), "adamw": list(self.adamw_names)}

    def free(self):
        self.engine.free()

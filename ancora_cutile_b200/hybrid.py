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


def _tileable(shape):
    """A 2-D shape the Newton-Schulz kernels can tile (both sides multiples of 128)."""
    return len(shape) == 2 and shape[0] % 128 == 0 and shape[1] % 128 == 0


def muon_names_for(shapes, is_muon=default_is_muon):
    """Names routed to Muon for a {name: shape} dict: ``is_muon`` and tileable (the rule
    ``HybridOptimizer`` applies, usable before any array exists)."""
    return [n for n, s in shapes.items()
            if is_muon(n, np.empty((0,) * len(s))) and _tileable(tuple(s))]


class _Part:
    """One sub-optimizer of the hybrid (the reference exposes ``.muon`` and ``.adamw`` as real
    optimizers, ancora/optim/hybrid.py:40-43).  Both parts share the engine's device arenas, so
    ``free()`` here releases nothing: ``HybridOptimizer.free()`` does."""

    def __init__(self, owner, kind, names, kw):
        self._o, self.kind, self.names, self.kw = owner, kind, names, kw
        self._steps = 0

    @property
    def lr(self):
        return self.kw["lr"]

    @lr.setter
    def lr(self, v):
        self.kw["lr"] = v

    @property
    def t(self):
        """Steps taken: the AdamW part's is the engine's step number (bias corrections, SR stream)."""
        return self._o.engine.t if self.kind == "adamw" else self._steps

    def step(self, grads, stream_int=None):
        """Steps only this part's tensors (grads: {name: ndarray} for this part's names)."""
        o = self._o
        si = stream_int if stream_int is not None else o.si
        e = o.engine
        e.upload_grads(o._expand(grads, self.names), si, kind=self.kind)
        e.step_part(self.kind, si)
        self._steps += 1
        e.ctx.sync(si)
        e.ctx.check_status()

    def weights(self):
        w = self._o.weights()
        return {n: w[n] for n in self.names}

    def master(self):
        m = self._o.master()
        return {n: m[n] for n in self.names if n in m}

    def free(self):
        pass


class HybridOptimizer:
    """Muon on 2-D hidden matrices + AdamW on everything else, with the reference's constructor
    and methods (ancora/optim/hybrid.py:28-56).

    Routing is ``is_muon(name, p)`` with two additions the device kernels need:
      * a 2-D tensor routed to Muon whose sides are not both multiples of 128 (a (1024, 16) MoE
        router, say) goes to AdamW instead of failing: the reference's host Muon takes any 2-D
        shape (optim/muon.py:287-318), its device classes assert like ours (muon.py:98);
        ``self.muon_fallback`` lists them;
      * ``expert_muon=True`` treats a 3-D stack (E, K, N) whose slices ``is_muon`` accepts as E
        Muon matrices, batched through one Newton-Schulz chain per shape (what the reference's
        resident MoE layer does, kernels/moe.py:567-609); by default a 3-D tensor goes to AdamW,
        as in the reference's host optimizer (moe_model.py:51-54).
    """

    def __init__(self, params, is_muon=default_is_muon, no_decay=None, muon_kw=None, adamw_kw=None,
                 si=None, muon_device=False, grad_dtype="f32", rounding="rne", seed=0,
                 rank=0, world=1, comm=None, schedule=None, max_batch=0, expert_muon=False, ctx=None):
        muon_kw = dict(lr=0.02, momentum=0.95, ns_steps=5, **(muon_kw or {}))
        adamw_kw = adamw_kw or dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.01)
        if no_decay is None:
            no_decay = lambda n, p: (p.ndim == 1)
        self.si = si
        routed = [n for n, p in params.items() if is_muon(n, p)]
        for n in routed:
            assert params[n].ndim == 2, f"Muon is for 2D matrices, {n} is {params[n].shape}"
        self.muon_fallback = [n for n in routed if not _tileable(params[n].shape)]
        self.muon_names = [n for n in routed if _tileable(params[n].shape)]
        # expert stacks: internal per-expert entries "name#e" over views of the caller's array
        self._stacks = {}
        if expert_muon:
            for n, p in params.items():
                if p.ndim == 3 and _tileable(p.shape[1:]) and is_muon(n, p[0]):
                    self._stacks[n] = int(p.shape[0])
                    self.muon_names.append(n)
        order = {n: i for i, n in enumerate(params)}
        self.muon_names.sort(key=order.get)
        self.adamw_names = [n for n in params if n not in set(self.muon_names)]
        eng_params, eng_muon, mset = {}, [], set(self.muon_names)
        for n, p in params.items():
            if n in self._stacks:
                for e in range(self._stacks[n]):
                    eng_params[f"{n}#{e}"] = p[e]
                    eng_muon.append(f"{n}#{e}")
            else:
                eng_params[n] = p
                if n in mset:
                    eng_muon.append(n)
        from .muon import _UNSET
        self.engine = ResidentHybrid(
            eng_params, eng_muon,
            no_decay_names=tuple(n for n in self.adamw_names if no_decay(n, params[n])),
            adamw_kw=adamw_kw, muon_kw=muon_kw, grad_dtype=grad_dtype, rounding=rounding, seed=seed,
            rank=rank, world=world, comm=comm, schedule=_UNSET if schedule is None else schedule,
            max_batch=max_batch, ctx=ctx)
        self.muon = _Part(self, "muon", self.muon_names, self.engine.muon_kw)
        self.adamw = _Part(self, "adamw", self.adamw_names, self.engine.adamw_kw)

    # ---- expert stacks <-> the engine's per-matrix entries
    def _expand(self, grads, names=None):
        """{caller's name: array} -> {engine entry: array}; slices of a stack are views."""
        if not self._stacks or grads is self.engine.pinned_grads():
            return grads
        out = {}
        for n in (grads if names is None else names):
            g = grads[n]
            if n in self._stacks:
                for e in range(self._stacks[n]):
                    out[f"{n}#{e}"] = g[e]
            else:
                out[n] = g
        return out

    def _collapse(self, per_entry, stack=np.stack):
        if not self._stacks:
            return per_entry
        out = {}
        for n, v in per_entry.items():
            base, sep, e = n.rpartition("#")
            if sep and base in self._stacks:
                if int(e) == 0:
                    out[base] = stack([per_entry[f"{base}#{k}"] for k in range(self._stacks[base])])
            else:
                out[n] = v
        return out

    def step(self, grads, stream_int=None):
        si = stream_int if stream_int is not None else self.si
        e = self.engine
        e.upload_grads(self._expand(grads), si)
        e.step(si)
        self.muon._steps += 1
        e.ctx.sync(si)
        e.ctx.check_status()

    def step_and_fetch(self, grads, stream_int=None):
        """step() and the read-back of the updated bf16 weights as ONE pipelined call: the
        gradient upload, the optimizer kernels and the download of finished parameters overlap
        unit by unit.  Returns {name: uint16 bf16 bit patterns} (views of page-locked memory,
        valid until the next call; a stack of experts comes back as one stacked copy)."""
        si = stream_int if stream_int is not None else self.si
        bits, _, _ = self.engine.step_host(self._expand(grads), si)
        self.muon._steps += 1
        self.engine.ctx.check_status()
        return self._collapse(bits)

    def pinned_grads(self):
        """Page-locked numpy views, one per parameter, that ``step`` / ``step_and_fetch`` copy
        from without an extra host copy when the caller writes gradients straight into them and
        passes this dict back.  Expert e of a stack ``name`` is the entry ``"name#e"``."""
        return self.engine.pinned_grads()

    def weights(self):
        """bf16-valued fp32 weights for the next forward, per name."""
        return self._collapse(self.engine.weights())

    def master(self):
        """fp32 masters per name (with ZeRO-1: only what this rank owns, owned range only)."""
        out = {}
        for n, (s, e, flat) in self.engine.master().items():
            full = int(np.prod(self.engine.shapes[n], dtype=np.int64))
            out[n] = flat.reshape(self.engine.shapes[n]) if (s, e) == (0, full) else flat
        if self._stacks and self.engine.world == 1:
            out = self._collapse(out)
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

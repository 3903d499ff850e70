"""Muon restated in numpy (test infrastructure; never on the product path).

Pieces and the reference lines they follow:

* ``PE_SCHEDULE`` / ``KELLER`` / ``coef_at``      ancora/kernels/muon_ns.py:21,30-42
* ``momentum``      nb = mu*b + g ; u = g + mu*nb  ancora/kernels/muon_ns.py:184-186
                                                  (host form: ancora/optim/muon.py:303-305)
* ``ns_fp32``       fp32 Newton-Schulz             ancora/optim/muon.py:67-80, with the
                    per-iteration schedule of tests/kernels/_probe_polar_express_device.py:29-36
* ``ns_bf16_chain`` the device chain's rounding points, fused form
                                                  ancora/kernels/muon_ns.py:245-276
* ``update``        pn = p - lr_scale*O ; p16=RNE  ancora/kernels/muon_ns.py:220-229
* ``shape_scale``   sqrt(max(1, rows/cols))        ancora/optim/muon.py:101,176,308
* ``host_muon_step`` the numpy optimizer          ancora/optim/muon.py:299-309
"""
import numpy as np

from .bf16 import rne_bits, rne_f32, bits_f32

KELLER = (3.4445, -4.7750, 2.0315)
PE_SCHEDULE = [(4.0848, -6.8946, 2.9270),
               (3.9505, -6.3029, 2.6377),
               (3.7418, -5.5913, 2.3037),
               (2.8769, -3.1427, 1.2046),
               (2.8366, -3.0525, 1.2012)]


def coef_at(schedule, k):
    if schedule is None:
        return KELLER
    return schedule[k] if k < len(schedule) else schedule[-1]


def shape_scale(rows, cols):
    return max(1.0, rows / cols) ** 0.5


def momentum(buf, g, mu):
    """Heavy-ball + Nesterov in float32.  Returns (new_buf f32, u f32 un-rounded)."""
    f = np.float32
    buf = np.asarray(buf, f); g = np.asarray(g, f); mu = f(mu)
    nb = mu * buf + g
    u = g + mu * nb
    return nb, u


def ns_fp32(G, steps=5, schedule=None, eps=1e-7):
    """fp32 Newton-Schulz on the orientation with rows <= cols; returns G's shape."""
    X = np.asarray(G, np.float32)
    tr = X.shape[0] > X.shape[1]
    if tr:
        X = X.T
    X = X / (np.linalg.norm(X) + eps)
    for k in range(steps):
        a, b, c = coef_at(schedule, k)
        A = X @ X.T
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X.T if tr else X


def fro_recip(Xf32, eps=1e-7):
    """1/(||X||_F + eps) in float32 from a float64 accumulation of the squares.

    The device kernel sums squares in float32 in a fixed tree; its result is
    compared with this one to a relative tolerance, not bitwise."""
    s = np.sqrt(np.sum(np.asarray(Xf32, np.float64) ** 2))
    return np.float32(1.0) / (np.float32(s) + np.float32(eps))


def ns_bf16_chain(X16, steps=5, schedule=None, eps=1e-7, recip=None):
    """Emulates the device chain on a (M,N) bf16-bit matrix with M <= N: every stored
    matrix (scaled X, A, B', Y) is rounded to bf16; products accumulate in higher
    precision and the combines happen before the rounding (fused epilogues).  As on the
    device, the a*X term rides in the polynomial's diagonal: B' = b A + c A A + a I and
    X' = B' X.  Tolerance-level model of the device result, used for error estimates only."""
    X = bits_f32(X16).astype(np.float32)
    if recip is None:
        recip = fro_recip(X, eps)
    X = rne_f32(X * np.float32(recip))
    for k in range(steps):
        a, b, c = (np.float32(t) for t in coef_at(schedule, k))
        A = rne_f32(X @ X.T)
        B = b * A + c * (A @ A)
        B[np.diag_indices_from(B)] += a
        X = rne_f32(rne_f32(B) @ X)
    return rne_bits(X)


def update(p, O16, lr_scale):
    """pn = p - lr_scale*f32(O) ; p16 = RNE(pn).  O16 are bf16 bits in p's orientation."""
    f = np.float32
    pn = np.asarray(p, f) - f(lr_scale) * bits_f32(O16)
    return pn, rne_bits(pn)


class HostMuon:
    """The reference's numpy Muon (ancora/optim/muon.py:287-318) with a coefficient
    schedule; schedule=None is the reference default (Keller)."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, schedule=None):
        self.lr, self.mom, self.nesterov, self.ns, self.schedule = lr, momentum, nesterov, ns_steps, schedule
        self.w = {n: np.asarray(p, np.float32).copy() for n, p in params.items()}
        self.buf = {n: np.zeros_like(w) for n, w in self.w.items()}

    def step(self, grads):
        for n, W in self.w.items():
            g = np.asarray(grads[n], np.float32)
            buf = self.buf[n]
            buf *= np.float32(self.mom)
            buf += g
            u = g + np.float32(self.mom) * buf if self.nesterov else buf
            o = ns_fp32(u, self.ns, self.schedule)
            W -= np.float32(self.lr * shape_scale(*W.shape)) * o

    def weights(self):
        return {n: rne_f32(W) for n, W in self.w.items()}

"""Thin Python wrappers over the kernel-level C entry points (one call = one or a
few kernel launches on the given stream, no synchronisation).  Arguments are device
buffers (anything ``dev_ptr`` accepts)."""
import ctypes as C

import numpy as np

from . import _lib as L
from .buffers import dev_ptr, get_context

_GRAD = {"bf16": L.GRAD_BF16, "f32": L.GRAD_F32}


def _coeff_array(coeffs):
    flat = [float(x) for t in coeffs for x in t]
    return (C.c_float * max(len(flat), 1))(*flat)


def ns_gemm_phase(mode, P, Q, Cout, E, M, N, alpha=0.0, beta=1.0, stream=None, ctx=None):
    """mode 0: C=RNE(P P^T); 1: C=RNE(alpha P + beta P P^T); 2: C=RNE(alpha Q + beta P Q)."""
    ctx = ctx or get_context()
    L.check(L.lib().anc_ns_gemm_phase(ctx.handle, int(mode), dev_ptr(P), dev_ptr(Q), dev_ptr(Cout),
                                      int(E), int(M), int(N), float(alpha), float(beta),
                                      C.c_void_p(stream or None)))


def muon_momentum(buf, g, u, K, N, momentum, nesterov=True, transposed=False, grad_dtype="bf16",
                  stream=None, ctx=None):
    ctx = ctx or get_context()
    L.check(L.lib().anc_muon_momentum(ctx.handle, dev_ptr(buf), dev_ptr(g), _GRAD[grad_dtype], dev_ptr(u),
                                      int(K), int(N), float(momentum), int(bool(nesterov)),
                                      int(bool(transposed)), C.c_void_p(stream or None)))


def muon_update(p32, p16, O, K, N, lr_scale, transposed=False, stream=None, ctx=None):
    ctx = ctx or get_context()
    L.check(L.lib().anc_muon_update(ctx.handle, dev_ptr(p32), dev_ptr(p16), dev_ptr(O), int(K), int(N),
                                    float(np.float32(lr_scale)), int(bool(transposed)),
                                    C.c_void_p(stream or None)))


def fro_normalize(X, recip, E, M, N, eps=1e-7, stream=None, ctx=None):
    ctx = ctx or get_context()
    L.check(L.lib().anc_fro_normalize(ctx.handle, dev_ptr(X), dev_ptr(recip), int(E), int(M), int(N),
                                      float(eps), C.c_void_p(stream or None)))


def ns_batched(X, A, B, Y, recip, E, M, N, steps, coeffs, eps=1e-7, stream=None, ctx=None, single_launch=True):
    """single_launch=False forces one launch per phase (same bits)."""
    ctx = ctx or get_context()
    L.check(L.lib().anc_ns_batched_ex(ctx.handle, dev_ptr(X), dev_ptr(A), dev_ptr(B), dev_ptr(Y),
                                      dev_ptr(recip), int(E), int(M), int(N), int(steps),
                                      _coeff_array(coeffs), float(eps), int(bool(single_launch)),
                                      C.c_void_p(stream or None)))


def grad_accumulate(acc, src=None, g16=None, numel=None, src_dtype="f32", elem_offset=0, scale=1.0,
                    rounding="rne", seed=0, step=0, zero_after=False, stream=None, ctx=None):
    """acc = src + acc (float32; src f32 or bf16, optional) and, in the same sweep,
    g16 = bf16(acc * scale) (optional; "rne" or "sr"), then acc = 0 when ``zero_after``.
    The accumulate sweep and the downcast the reference runs separately
    (ancora/kernels/fused.py:242-249, 144-161)."""
    ctx = ctx or get_context()
    if numel is None:
        numel = int(np.prod(acc.shape))
    L.check(L.lib().anc_grad_accumulate(ctx.handle, dev_ptr(acc), dev_ptr(src), _GRAD[src_dtype], dev_ptr(g16),
                                        int(numel), int(elem_offset), float(np.float32(scale)),
                                        {"rne": L.ROUND_RNE, "sr": L.ROUND_SR}[rounding], int(seed), int(step),
                                        int(bool(zero_after)), C.c_void_p(stream or None)))
